"""Wall-clock phase stamps of one CTA of the two decode GEMV kernels (diagnostics; not part of the library).

The library records the stamps when the context option "tc_trace" is 1 (CTA 0 writes %globaltimer values into the
tail of the context workspace; ribn_debug_read_trace copies them out).  Usage, from the repository root:

    python tests/probes/pipeline_trace.py FORMAT N K MEMBERS        e.g.  12 12288 4096 1   (Q4_K, one row: integer-dot kernel)
                                                                          12 12288 4096 16  (tensor-core decode kernel)
Twelve launches over twelve distinct weight copies run first, so the traced launch is L2-cold.
"""
import os
import sys

import numpy as np
import torch

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", ".."))
import engine_b200  # noqa: E402
from engine_b200 import synth  # noqa: E402


def main():
    fmt, n, k, m = (int(v) for v in sys.argv[1:5])
    ctx = engine_b200.RibnContext(0)
    ctx.set_option("tc_trace", 1)
    if len(sys.argv) > 5:
        ctx.set_option("tc_ksplit", int(sys.argv[5]))
    copies = [engine_b200.CudaQuantizedWeight(engine_b200.WeightTensorSpec.new("w", [k, n]), fmt,
                                              synth.random_weight_device(fmt, k, n, i, ctx.device)) for i in range(12)]
    x = torch.randn(m, k, device=ctx.device).to(torch.bfloat16)
    y = torch.empty(m, n, device=ctx.device)
    kernel = engine_b200.QwenGemvKernel.from_value_type(fmt, ctx)
    for w in copies:
        kernel.execute_warp_batch(w, x, y, m)
    ctx.synchronize()
    buf = np.zeros(4 * 64 * 8, np.int64)
    ctx.check(ctx._lib.ribn_debug_read_trace(ctx.handle, buf.ctypes.data, buf.nbytes))
    print(f"format {fmt}, {n}x{k}, {m} member rows; last of 12 cold launches, CTA 0; microseconds after kernel entry")
    if m <= 4:   # integer-dot kernel: flat event list
        t0 = buf[0]
        for event, name in ((1, "producer: first ring of weight stages requested"), (2, "producer: past the dependency wait"),
                            (3, "consumers: packed activations landed")):
            if buf[event]:
                print(f"  {name:48s} {(buf[event] - t0) / 1e3:7.2f}")
        for it in range(12):
            if buf[8 + 2 * it]:
                print(f"  stage {it:2d}: data seen {(buf[8 + 2 * it] - t0) / 1e3:7.2f}   consumed {(buf[9 + 2 * it] - t0) / 1e3:7.2f}")
        for tile in range(8):
            if buf[40 + tile]:
                print(f"  tile {tile}: outputs stored {(buf[40 + tile] - t0) / 1e3:7.2f}")
        print(f"  {'consumer thread 0 done':48s} {(buf[4] - t0) / 1e3:7.2f}")
    else:        # tensor-core decode kernel: wall stamps live in row (role 3, step 63)
        t = buf.reshape(4, 64, 8)[3, 63]
        names = ["kernel entry", "after the prologue barrier", "activation warp past the dependency wait", "first MMA group ready",
                 "last MMA group ready", "accumulation done", "teardown"]
        for i, name in enumerate(names):
            print(f"  {name:48s} {(t[i] - t[0]) / 1e3:7.2f}")


if __name__ == "__main__":
    main()
