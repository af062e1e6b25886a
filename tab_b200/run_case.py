"""Run one operator of the library on synthetic data and print its time (a small, fixed-size case for
profilers and quick measurements).

    python -m tab_b200.run_case conv     --type 0 --N 64 --H 56 --C 64 --KN 64 --K 3 --stride 1 --pad 1
    python -m tab_b200.run_case packed   ...        # the popcount convolution alone on pre-packed activations
    python -m tab_b200.run_case bits     ...        # the tensor-core GEMM stage alone (bit-planes + prepared byte weights);
                                                    # --chain / --residual / --int16 select its epilogue
    python -m tab_b200.run_case quantize --bitwidth 2 --N 256 --H 56 --C 256

Prints one JSON line: milliseconds per call (CUDA events, after warm-up) and the derived TOPS or GB/s.
"""
from __future__ import annotations

import argparse
import json

import torch

from . import ops


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("op", choices=["conv", "packed", "bits", "quantize", "probe"])
    ap.add_argument("--kind", type=int, default=0, help="probe: 0 POPC, 1 LOP3, 2 s8 mma.sync, 3 b1 mma and.popc, 4 b1 mma xor.popc")
    ap.add_argument("--type", type=int, default=0)
    ap.add_argument("--bitwidth", type=int, default=2)
    ap.add_argument("--N", type=int, default=64)
    ap.add_argument("--H", type=int, default=56)
    ap.add_argument("--C", type=int, default=64)
    ap.add_argument("--KN", type=int, default=64)
    ap.add_argument("--K", type=int, default=3)
    ap.add_argument("--stride", type=int, default=1)
    ap.add_argument("--pad", type=int, default=1)
    ap.add_argument("--iters", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=2)
    ap.add_argument("--residual", action="store_true", help="bits: add a residual tensor in the epilogue")
    ap.add_argument("--chain", action="store_true", help="bits: per-image sums of |y| and the next layer's thresholds in the epilogue")
    ap.add_argument("--int16", action="store_true", help="bits: 16-bit integer output (the hand-over to the next quantiser)")
    ap.add_argument("--path", type=int, default=0, help="conv: 0 tensor cores, 1 popcount kernel, 2 popcount kernel, one POPC per word")
    a = ap.parse_args()
    dev = torch.device("cuda:0")
    from . import _cabi
    _cabi.lib().tab_conv2d_set_path(a.path)
    torch.manual_seed(0)
    if a.op == "probe":
        import ctypes
        l = _cabi.lib()
        sink = torch.empty(l.tab_pipe_probe_sink_bytes(), dtype=torch.uint8, device=dev)
        n_ops = ctypes.c_double(0)
        best = None
        for i in range(a.iters + a.warmup):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            _cabi.check(l.tab_pipe_probe_launch(a.kind, 2048, sink.data_ptr(), ctypes.byref(n_ops), torch.cuda.current_stream().cuda_stream), "probe")
            e1.record()
            torch.cuda.synchronize()
            if i >= a.warmup:
                ms = e0.elapsed_time(e1)
                best = ms if best is None else min(best, ms)
        print(json.dumps({"op": "probe", "kind": a.kind, "ms": best, "value": n_ops.value / best / 1e9, "unit": "Gop/s (lane instructions, or binary/int8 ops for the MMA kinds)"}))
        return
    N, H, W, C, KN, K, s, p, t = a.N, a.H, a.H, a.C, a.KN, a.K, a.stride, a.pad, a.type
    x = torch.randn(N, H, W, C, device=dev)
    ths = (0.7 * x.abs().mean(dim=(1, 2, 3))).contiguous()
    if a.op == "quantize":
        fn = lambda: ops.Quantize(x, ths, a.bitwidth, N, H, W, C)
        bits = 1 if a.bitwidth == 1 else 2
        work = 4 * N * H * W * C + 8 * N * H * W * ((C + 63) // 64) * bits + 8 * N
        unit, scale = "GB/s", 1e6
    else:
        w = torch.randn(KN, K, K, C, device=dev)
        wths = (0.7 * w.abs().mean(dim=(1, 2, 3))).contiguous()
        qw, btn = ops.Quantize(w, wths, 1 if t in (1, 3) else 2, KN, K, K, C)
        oh = (H + 2 * p - K + 1) // s
        work = 2 * N * oh * oh * KN * K * K * C
        unit, scale = "TOPS", 1e9
        if a.op == "conv":
            fn = lambda: ops.Conv2d(x, qw, ths, btn, t, p, p, s, s, N, H, W, C, KN, K, K)
        else:
            qx, _ = ops.Quantize(x, ths, 1 if t in (2, 3) else 2, N, H, W, C)
            if a.op == "bits":
                w8 = ops.expand_weights(qw, 1 if t in (1, 3) else 2, KN, K, K, C)
                res = torch.round(torch.randn(N, KN, oh, oh, device=dev) * 8) if a.residual else None
                state = ops.new_state(N, dev) if a.chain else None
                fn = lambda: ops.conv2d_bits(qx, w8, t, p, p, s, s, N, H, W, C, KN, K, K, residual=res,
                                             threshold_scale=0.7 if a.chain else None, state=state, out_int16=a.int16)
            else:
                fn = lambda: ops.conv2d_packed(qx, qw, btn, t, p, p, s, s, N, H, W, C, KN, K, K)
    for _ in range(a.warmup):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(a.iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / a.iters
    print(json.dumps({"op": a.op, "args": vars(a), "ms": ms, "value": work / ms / scale, "unit": unit,
                      "kernel": _cabi.lib().tab_last_conv_kernel().decode(), "device_status": _cabi.lib().tab_device_status()}))


if __name__ == "__main__":
    main()
