// Activation packer for the integer-dot GEMV, with the RMSNorm that precedes
// the projections optionally fused in.
//
//   (x [members][K], f32 or bf16)  ->  per member: q1[kpad] | q2[kpad] | dq[kpad/32] | sum[kpad/32]
//
// Per block of 32 values: d = the power of two at or above max|x|/127,
// q1 = round(x/d), q2 = round((x - q1*d) * 256/d), dq = d/256, so that
// x ~= dq * (256*q1 + q2) with an error of at most d/512 <= max|x|/32512.
// A power-of-two step makes the split exact whenever the values carry at most
// ~14 bits below the block maximum: bf16 activations near the block maximum and
// every fixture built from dyadic values reproduce exactly.  `sum` is the f32
// sum of the block's values (the multiplier of the Q4_K / Q5_K group minimum).
//
// Role in the reference: the counterpart of CudaQ8_1Quantizer / quantize_q8_1
// (crates/nvidia/src/activation.cu:3-28, activation.rs:15-88), which packs one
// int8 plane with f16 scale and sum and is lossy at the 1e-2 level; this packer
// keeps two planes and f32 scale and sum.  With norm_weight it also replaces
// the rms_norm launch in front (crates/nvidia/src/model_ops.rs:106-199): one CTA
// per row reduces sum(x^2), then packs x * inv_rms * norm_weight.
#include <cuda_bf16.h>

#include "internal.h"
#include "pack_activations.cuh"
#include "pipeline.cuh"

namespace ribn {
namespace {

constexpr int kPackThreads = 512;

// One CTA per member row.  Thread t owns the 8-element chunks t, t + 512, ...; four consecutive
// threads share a block of 32 and combine their maxima and sums with two shuffles.
template <typename XT>
__global__ void __launch_bounds__(kPackThreads) quantize_activations_kernel(const XT* __restrict__ x, int mode,
                                                                            const float* __restrict__ norm_weight, float eps,
                                                                            uint8_t* __restrict__ packed, int k, int kpad) {
    __shared__ float partial[kPackThreads / 32];
    pdl_launch_dependents();
    pdl_wait_prior();   // x may be the previous kernel's output; the packed rows may still be read by it
    const XT* xr = x + static_cast<size_t>(blockIdx.x) * k * (mode == 2 ? 2 : 1);
    uint8_t* out = packed + static_cast<size_t>(blockIdx.x) * packed_activation_stride(kpad);
    pack_activation_row<kPackThreads>(xr, mode, norm_weight, eps, out, k, kpad, partial, static_cast<int>(threadIdx.x),
                                      [] { __syncthreads(); });
}

template <typename XT>
cudaError_t launch(const void* x, const float* norm_weight, float eps, void* packed, int members, int k, int kpad,
                   bool swiglu, cudaStream_t stream) {
    const int mode = swiglu ? 2 : (norm_weight != nullptr ? 1 : 0);
    return launch_kernel(quantize_activations_kernel<XT>, dim3(members), dim3(kPackThreads), 0, stream, static_cast<const XT*>(x), mode,
                         norm_weight, eps, static_cast<uint8_t*>(packed), k, kpad);
}

}  // namespace

cudaError_t launch_quantize_activations(const void* x, bool x_bf16, const float* norm_weight, float eps, void* packed,
                                        int members, int k, cudaStream_t stream, bool swiglu) {
    const int kpad = padded_k(k);
    return x_bf16 ? launch<__nv_bfloat16>(x, norm_weight, eps, packed, members, k, kpad, swiglu, stream)
                  : launch<float>(x, norm_weight, eps, packed, members, k, kpad, swiglu, stream);
}

}  // namespace ribn
