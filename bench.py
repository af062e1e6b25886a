#!/usr/bin/env python3
"""Benchmark of the TAB hot path on B200: binary-op TOPS of ``TAB_Conv2d`` (and HBM GB/s of
``TAB_Quantize``), one JSON line on stdout.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
           --master-port P bench.py --gpus N --steps K --warmup W

Workload (synthetic, seeded): the ResNet-18-shaped ternary (TNN) chain of ``tab_b200.chain`` - 16 3x3 and
3 1x1 convolutions, global batch 256 of 56x56x64 fp32 NHWC activations, random N(0,1) weights
ternarised at 0.7*mean|w| per filter, per-image thresholds 0.7*mean|x| recomputed before every
convolution.  One step = one forward of the whole batch.  With N GPUs the batch is sharded (256/N images
per GPU, weights replicated) and the fp32 outputs are all-gathered over NCCL inside the timed region:
total work is fixed, i.e. strong scaling.

binary-ops = 2*M*KN*KH*KW*C summed over the convolutions (0.868e12 per step); every other kernel in the
step (activation quantise, residual add, thresholds) counts as time but not as ops.

``value``   device-resident input, CUDA-event time of the K steps, L2 flushed between steps, max over ranks.  The chain runs
            on prepared convolutions (``tab_b200.nn.TABConv2d``: weights quantised and byte-expanded once, as an inference
            caller holds them): per convolution input one ``tab_quantize_launch`` (fp32 -> bit-planes, shared by a block's
            first convolution and its shortcut) and per convolution one ``tab_conv2d_bits_launch`` (persistent tcgen05
            kernel; residual, |y| sums and the next thresholds in its epilogue).
``e2e``     the same step through the TAB_CUDA extension module with the input in pinned host memory: the host-to-device
            copy of the shard and the device-to-host copy of the output are inside the timed region.  The shard is processed
            in chunks of images so that the copies of one chunk overlap the forward of another.
``roofline`` the whole step against HBM (the fp32-in / fp32-out operator interface makes the step byte-bound: algorithmic bytes
            of every launch, summed, over ``ms_per_step``), with the GEMM stage alone against the tensor pipe
            (``gemm_stage``, denominator measured in the same run by the library's tcgen05 issue probe), ``TAB_Quantize``
            alone against HBM (``quantize``) and the bit-packed popcount kernel against the integer pipes (``popcount``).
``parity_check`` (inside ``config``) after the timed loops the outputs of sampled images (at N > 1: one image of every
            rank's shard, taken from the gathered tensor) are compared bit for bit with the CPU oracle chain run on the
            input thresholds the GPU computed; a mismatch makes the run exit non-zero.
``cpu_baseline`` / ``--impl reference``: the reference's CPU algorithm (quantise, pad, im2row, its own
            compiled *GEMM_baseline functions when oracle/_ref exists, else the C port) on the host cores,
            on a bounded sample of images of the same workload.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import numpy as np  # noqa: E402

GLOBAL_BATCH = 256
H0 = W0 = 56
C0 = 64
CONV_TYPE = 0
WEIGHT_SEED = 5000
INPUT_SEED = 5
# dram__bytes_read.sum + dram__bytes_write.sum per image of the step's largest launch, conv_umma_persist_kernel<2,64,6,1,2,1>
# (56x56x64 -> 64 with residual and next thresholds), from the ncu capture summarised under profiles/: 54.72 MB read +
# 10.07 MB written at 64 images.  The bytes read (residual + bit-planes) are proportional to the images; of the 51.4 MB of
# output only 10 MB had left the 126 MB L2 when that small launch ended, so the scaled figure is a lower bound for a launch
# whose output exceeds the L2 (algorithmic: 1.66 MB per image, of which 0.80 MB output).
L1_TRAFFIC_PER_IMAGE = (54.720256e6 + 10.072832e6) / 64


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--cpu-sample-images", type=int, default=32)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-layer-table", action="store_true")
    ap.add_argument("--sustained-seconds", type=float, default=2.0)
    return ap.parse_args()


def workload_config(n_gpus):
    from tab_b200 import chain
    return {"workload": "resnet18-shaped TNN chain: 16x conv3x3 + 3x conv1x1 (s2,p0), 56x56x64 -> 7x7x512, type 0",
            "global_batch": GLOBAL_BATCH, "per_gpu_batch": GLOBAL_BATCH // max(n_gpus, 1), "input": "fp32 NHWC N(0,1)",
            "thresholds": "0.7*mean|.| per image / per filter", "parallelism": "dp%d (batch sharded, weights replicated, NCCL all-gather of outputs)" % n_gpus,
            "l2": "flushed between timed steps (256 MiB write)", "binary_ops_per_step": chain.chain_binary_ops(GLOBAL_BATCH)}


# ------------------------------------------------------------------------------------------------
# CPU arm (the only place this file touches oracle/)
# ------------------------------------------------------------------------------------------------

def host_threads():
    """Threads the CPU arm uses: every core this process may run on, set explicitly in the OpenMP runtime, so that a
    launcher's OMP_NUM_THREADS=1 (torch.distributed.run exports it for more than one process per node) does not apply."""
    from oracle import c_oracle
    n = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
    c_oracle.omp_threads(n, "v3")
    c_oracle.omp_threads(n, "shipped")
    return n


def cpu_chain_once(sample_images, variant, use_ref, x=None, qweights=None, ths=None):
    from oracle.oracle_ops import OracleOps
    from oracle import c_oracle
    from tab_b200 import chain

    class Ops(OracleOps):
        @staticmethod
        def Conv2d(x_, qw, ths_, btn, t, p1, p2, s1, s2, N, H, W, C, KN, KH, KW):
            return c_oracle.conv2d(np.asarray(x_).reshape(-1), qw, ths_, btn, t, p1, p2, s1, s2, N, H, W, C, KN, KH, KW,
                                   use_ref_gemm=use_ref, variant=variant)

    if x is None:
        rng = np.random.default_rng(INPUT_SEED)
        x = rng.standard_normal((sample_images, H0, W0, C0), dtype=np.float32)
    if qweights is None:
        qweights = chain.quantize_weights(chain.make_weights(WEIGHT_SEED, CONV_TYPE), CONV_TYPE, OracleOps.Quantize)
    t0 = time.perf_counter()
    if ths is None:
        ths = OracleOps.residual_threshold(x.copy(), None, chain.THRESHOLD_SCALE)
    y, _, _, _ = chain.forward(Ops, x, ths, qweights, CONV_TYPE, sample_images)
    dt = time.perf_counter() - t0
    return dt, x, qweights, y


def cpu_baseline(sample_images, repeats=2):
    """Time the CPU pipeline on `sample_images` images of the workload.  Returns the JSON object."""
    threads = host_threads()
    from oracle import build, c_oracle
    from tab_b200 import chain
    build.build_oracle()
    build.build_ref()       # no-op without the reference tree; prebuilt libraries are used if present
    use_ref = c_oracle.ref_available("v3")
    ops = chain.chain_binary_ops(sample_images)
    out = {}
    x = qw = None
    for variant in ("v3", "shipped"):
        best = None
        for _ in range(repeats if variant == "v3" else 1):
            dt, x, qw, _ = cpu_chain_once(sample_images, variant, use_ref and c_oracle.ref_available(variant), x, qw)
            best = dt if best is None else min(best, dt)
        out[variant] = ops / best / 1e12
    used = c_oracle.omp_threads()
    return {
        "value": out["v3"], "unit": "TOPS", "cores": used,
        "kind": "reference" if use_ref else "port",
        "sample": "%d of %d images of the same chain (all 19 convolutions, thresholds and residuals included); "
                  "OpenMP, %d threads (omp_get_max_threads; %d cores available); GEMM stage = %s; flags of the reference's Setup_GCC.py "
                  "plus -march=x86-64-v3 (as-shipped flags: %.4f TOPS)" % (sample_images, GLOBAL_BATCH, used, threads,
                                                                          "the reference's compiled *GEMM_baseline" if use_ref else "C port of it",
                                                                          out["shipped"]),
        "as_shipped_flags_value": out["shipped"],
    }


def run_reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    threads = host_threads()
    from oracle import build, c_oracle
    from tab_b200 import chain
    build.build_oracle()
    build.build_ref()
    use_ref = c_oracle.ref_available("v3")
    S = args.cpu_sample_images
    ops = chain.chain_binary_ops(S)
    x = qw = None
    for _ in range(max(args.warmup, 1)):
        _, x, qw, _ = cpu_chain_once(S, "v3", use_ref, x, qw)
    t = 0.0
    for _ in range(args.steps):
        dt, x, qw, _ = cpu_chain_once(S, "v3", use_ref, x, qw)
        t += dt
    used = c_oracle.omp_threads()
    val = ops * args.steps / t / 1e12
    sample = ("each step = %d of %d images of the chain on the host cores (OpenMP, %d threads by omp_get_max_threads, %d cores available); "
              "GEMM stage = %s; Setup_GCC.py flags + -march=x86-64-v3" % (S, GLOBAL_BATCH, used, threads,
                                                                         "reference *GEMM_baseline (oracle/_ref)" if use_ref else "C port"))
    line = {
        "impl": "reference", "metric": "TAB_Conv2d binary-op TOPS", "value": val, "unit": "TOPS",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": t / args.steps * 1e3,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "u64 popcount", "data": "synthetic",
        "config": workload_config(args.gpus),
        "cpu_baseline": {"value": val, "unit": "TOPS", "cores": used, "kind": "reference" if use_ref else "port", "sample": sample},
        "e2e": {"value": val, "unit": "TOPS", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    emit(line)


def oracle_chain_images(x_images, ths_images):
    """The CPU oracle chain on a few images with given input thresholds (every later threshold follows from the data)."""
    from oracle.oracle_ops import OracleOps
    from tab_b200 import chain
    qweights = chain.quantize_weights(chain.make_weights(WEIGHT_SEED, CONV_TYPE), CONV_TYPE, OracleOps.Quantize)
    y, _, _, _ = chain.forward(OracleOps, np.ascontiguousarray(x_images), np.ascontiguousarray(ths_images), qweights, CONV_TYPE, x_images.shape[0])
    return np.asarray(y).reshape(x_images.shape[0], -1)


# ------------------------------------------------------------------------------------------------
# GPU arm
# ------------------------------------------------------------------------------------------------

class ClockSampler:
    """nvidia-smi in the background during the timed region (read-only queries)."""
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, uuid):
        self.uuid = uuid
        self.proc = None
        self.path = None

    def start(self):
        try:
            fd, self.path = tempfile.mkstemp(prefix="tab_clocks_", suffix=".csv")
            os.close(fd)
            self.proc = subprocess.Popen(["nvidia-smi", "-i", self.uuid, "--query-gpu=" + self.FIELDS,
                                          "--format=csv,noheader,nounits", "-lms", "20"],
                                         stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self):
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        if self.proc is None:
            return out
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, pw, reasons = [], [], [], set()
        try:
            for ln in open(self.path):
                f = [v.strip() for v in ln.split(",")]
                if len(f) < 7:
                    continue
                try:
                    sm.append(float(f[0])); mx.append(float(f[1])); pw.append(float(f[2]))
                except ValueError:
                    continue
                for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[3:7]):
                    if v.lower().startswith("active"):
                        reasons.add(name)
            os.unlink(self.path)
        except Exception:
            pass
        if sm:
            # under load = the samples drawing the most power (the sampler also sees the gaps between steps)
            order = sorted(range(len(sm)), key=lambda i: pw[i])[len(sm) // 2:]
            out.update(sm_mhz=statistics.median([sm[i] for i in order]), sm_max_mhz=max(mx), reasons=sorted(reasons), samples=len(sm),
                       power_w_max=max(pw))
        return out


def step_algorithmic_bytes(n_images):
    """Bytes every launch of one step must move, summed: per convolution input its elements read (4 B each; 2 B where the
    producer handed it over as int16) and 2 bits/element written by the quantiser; per convolution those bit-planes read, the
    byte weights read, the output written (4 B/element; 2 B for a block's first convolution, whose only reader is the next
    quantiser) and, where a shortcut is added, 4 B/element of residual read; the input statistics pass reads x once."""
    from tab_b200 import chain
    total = 4 * n_images * H0 * W0 * C0
    h = H0
    for b in chain.resnet18_blocks():
        a, bb, sc = b.conv_a, b.conv_b, b.shortcut
        oh = (h + 2 * a.pad - a.K + 1) // a.stride
        x_el, y_el = n_images * h * h * a.C, n_images * oh * oh * a.KN
        bits_in, bits_mid = x_el // 4, y_el // 4
        total += 4 * x_el + bits_in                                        # quantise x
        total += bits_in + a.KN * 9 * a.C + 2 * y_el                       # conv_a, int16 out
        if sc is not None:
            total += bits_in + sc.KN * sc.C + 4 * y_el                     # shortcut on the same bit-planes
        total += 2 * y_el + bits_mid                                       # quantise y1 (int16)
        total += bits_mid + bb.KN * 9 * bb.C + 4 * y_el + 4 * y_el         # conv_b + residual
        h = oh
    return total


_JSON_FD = None


def emit(line):
    """The one JSON line, on the real stdout."""
    data = (json.dumps(line) + "\n").encode()
    if _JSON_FD is None:
        sys.stdout.write(data.decode())
        sys.stdout.flush()
    else:
        os.write(_JSON_FD, data)


def main():
    global _JSON_FD
    args = parse_args()
    # stdout carries the JSON line and nothing else: whatever libraries print there from native code (NCCL announces its
    # version on stdout) is sent to stderr
    sys.stdout.flush()
    _JSON_FD = os.dup(1)
    os.dup2(2, 1)
    if args.impl == "reference":
        run_reference_arm(args)
        return

    import ctypes
    import torch
    import torch.distributed as dist
    from tab_b200 import _cabi, chain, dp, nn as tab_nn, ops as tab_ops

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU fallback)")
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus and world == 1 and args.gpus > 1:
        raise SystemExit("launch with torch.distributed.run --nproc-per-node %d for --gpus %d" % (args.gpus, args.gpus))
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    lib = _cabi.lib()
    import TAB_CUDA  # the reference-facing extension module (built in-tree by Setup_CUDA.py)

    N = GLOBAL_BATCH
    lo, hi = dp.shard_bounds(N, world, rank)
    n_local = hi - lo

    # ---- synthetic data: identical on every rank, each rank keeps its shard -------------------------
    gen = torch.Generator(device="cpu")
    gen.manual_seed(INPUT_SEED)
    x_host_full = torch.randn(N, H0, W0, C0, generator=gen)
    x_host = x_host_full[lo:hi].contiguous().pin_memory()
    x_dev = x_host.to(dev)
    weights = chain.make_weights(WEIGHT_SEED, CONV_TYPE)
    specs = {cs.name: cs for cs in chain.conv_specs()}
    launches = [0]

    class CountingConv(tab_nn.TABConv2d):
        """tab_b200.nn.TABConv2d with a kernel-launch counter (quantize = one kernel, conv_bits = one kernel)."""
        def quantize(self, x, thresholds=None):
            launches[0] += 1
            return super().quantize(x, thresholds)

        def conv_bits(self, *a, **k):
            launches[0] += 1
            out = super().conv_bits(*a, **k)
            # the quantised hand-over to the next layer comes from the same kernel ("+next") or from a quantiser launch behind it
            if k.get("next_bitwidth") is not None and "+next" not in lib.tab_last_conv_kernel().decode():
                launches[0] += 1
            return out

    class ModuleConv:
        """The same prepared convolution through the TAB_CUDA extension module."""
        def __init__(self, conv):
            self.c = conv
            wb = tab_nn.weight_bitwidth(conv.conv_type)
            self.W8 = TAB_CUDA.ExpandWeights(conv.QW, wb, conv.KN, conv.KH, conv.KW, conv.C)
            self.state = None
            self.conv_type = conv.conv_type

        def quantize(self, x, thresholds):
            n, h, w = (int(v) for v in x.shape[:3])
            ab = tab_nn.act_bitwidth(self.c.conv_type)
            if x.dtype == torch.int16:
                return TAB_CUDA.QuantizeI16(x, thresholds, ab, n, h, w, self.c.C)
            return TAB_CUDA.Quantize(x, thresholds, ab, n, h, w, self.c.C)[0]

        def conv_bits(self, QX, n, h, w, residual, scale, out_int16=False, next_bitwidth=None):
            if scale is not None and (self.state is None or self.state.numel() < lib.tab_conv2d_state_bytes(n)):
                self.state = TAB_CUDA.NewState(QX, n)
            out = TAB_CUDA.Conv2dBits(QX, self.W8, self.c.conv_type, *self.c.geometry(n, h, w), residual,
                                      self.state if scale is not None else None, scale if scale is not None else 0.0, bool(out_int16),
                                      int(next_bitwidth or 0))
            y = out[0]
            res = (y.view(n, y.shape[2], y.shape[3], y.shape[1]), (out[1] if scale is not None else None))
            return res + (out[2],) if next_bitwidth else res

    def nhwc(y):                                             # Conv2d's {N,KN,OH,OW} label over the [N][OH][OW][KN] buffer
        return y.view(y.shape[0], y.shape[2], y.shape[3], y.shape[1])

    class NhwcConv(CountingConv):
        def conv_bits(self, *a, **k):
            out = super().conv_bits(*a, **k)
            return (nhwc(out[0]),) + tuple(out[1:])

    convs = {}
    for name, (w, t) in weights.items():
        cs = specs[name]
        convs[name] = NhwcConv.from_float(torch.from_numpy(w).to(dev), CONV_TYPE, cs.pad, cs.stride, torch.from_numpy(t).to(dev), chain.THRESHOLD_SCALE)
    mconvs = {k: ModuleConv(v) for k, v in convs.items()}
    flush_buf = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    ops_per_step = chain.chain_binary_ops(N)
    per_img_out = 7 * 7 * 512

    y_full = torch.empty(N * per_img_out, dtype=torch.float32, device=dev)
    y_host = torch.empty(N * per_img_out, dtype=torch.float32).pin_memory() if rank == 0 else None

    first_conv = chain.resnet18_blocks()[0].conv_a.name

    def forward(cset, x_in, nb, count=True):
        if cset is convs:
            # thresholds of the chain's input and its bit-planes from one launch
            if count:
                launches[0] += 1
            qx0, ths = convs[first_conv].quantize_auto(x_in)
            y, _, _, _ = chain.forward_prepared(cset, x_in, ths, nb, compact_mid=True, fused_quant=True, qx0=qx0)
            return y, ths
        if count:
            launches[0] += 2
        ths = tab_ops.residual_threshold(x_in.reshape(nb, -1), None, chain.THRESHOLD_SCALE)      # reduce + finalise kernels
        y, _, _, _ = chain.forward_prepared(cset, x_in, ths, nb, compact_mid=True, fused_quant=True)
        return y, ths

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, steps, flush=True):
        evs = []
        for _ in range(steps):
            if flush:
                flush_buf.fill_(1)                  # L2 flush: 256 MiB write, outside the timed events
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            evs.append((e0, e1))
        torch.cuda.synchronize()
        return sum(a.elapsed_time(b) for a, b in evs)

    def max_over_ranks(v):
        if world == 1:
            return v
        t = torch.tensor([v], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    # ---- CUDA graph of one forward (the step is ~32 short launches: replaying a graph removes the launch
    #      gaps; the library's launches take a stream and never allocate or synchronise, so they capture) ----
    def make_graph(cset, x_static, nb):
        try:
            side = torch.cuda.Stream(dev)
            side.wait_stream(torch.cuda.current_stream(dev))
            with torch.cuda.stream(side):
                for _ in range(2):                       # first calls set kernel attributes and look up symbols: outside capture
                    forward(cset, x_static, nb, count=False)
            torch.cuda.current_stream(dev).wait_stream(side)
            torch.cuda.synchronize()
            gr = torch.cuda.CUDAGraph()
            with torch.cuda.graph(gr):
                y, ths = forward(cset, x_static, nb, count=False)
            return gr, y, ths
        except Exception as exc:                          # report and fall back to eager launches
            sys.stderr.write("cuda graph capture failed (%s): timing eager launches\n" % exc)
            return None, None, None

    # End-to-end step: the shard is processed in NCH chunks of images (every image is independent), so that the
    # host-to-device copy of chunk i+1 overlaps the forward of chunk i: input buffers / graphs in rotation,
    # copies on their own streams.
    # (Half-size chunks at the end, to shorten the forward that follows the last copy, measured slower: a forward of 16
    # images takes 0.8 of the time of one of 32.)
    NCH = 8 if n_local % 8 == 0 and n_local >= 64 else (4 if n_local % 4 == 0 and n_local >= 16 else 1)
    nb_e2e = n_local // NCH
    chunk_sizes = [nb_e2e] * NCH
    chunk_lo = [sum(chunk_sizes[:i]) for i in range(len(chunk_sizes))]
    NBUF = 3 if len(chunk_sizes) > 2 else len(chunk_sizes)
    x_chunk = [torch.empty((nb_e2e, H0, W0, C0), dtype=torch.float32, device=dev) for _ in range(NBUF)]
    y_local = torch.empty(n_local * per_img_out, dtype=torch.float32, device=dev)
    g_dev = make_graph(convs, x_dev, n_local)
    # one graph per (input buffer, chunk size) pair the schedule uses
    g_e2e = {}
    for i, sz in enumerate(chunk_sizes):
        k = i % NBUF
        if (k, sz) not in g_e2e:
            g_e2e[(k, sz)] = make_graph(mconvs, x_chunk[k][:sz], sz)
    use_graph = g_dev[0] is not None and all(g[0] is not None for g in g_e2e.values())
    h2d_stream = torch.cuda.Stream(dev)
    d2h_stream = torch.cuda.Stream(dev)
    launches[0] = 0
    forward(convs, x_dev, n_local)                        # count one forward's kernels
    launches_per_step = launches[0]
    torch.cuda.synchronize()

    def finish(y, gather=True):
        if world > 1 and gather:
            dist.all_gather_into_tensor(y_full, y.reshape(-1))
            return y_full
        return y.reshape(-1)

    def step_value(gather=True):
        if use_graph:
            g_dev[0].replay()
            return finish(g_dev[1], gather)
        return finish(forward(convs, x_dev, n_local)[0], gather)

    def step_e2e():
        main_s = torch.cuda.current_stream(dev)
        h2d_stream.wait_stream(main_s)               # the step starts where the caller's stream is
        ev_in, ev_done = [], []
        for i, sz in enumerate(chunk_sizes):
            k = i % NBUF
            with torch.cuda.stream(h2d_stream):
                if i >= NBUF:
                    h2d_stream.wait_event(ev_done[i - NBUF])             # the buffer's previous chunk has been consumed
                x_chunk[k][:sz].copy_(x_host[chunk_lo[i]:chunk_lo[i] + sz], non_blocking=True)
                e = torch.cuda.Event(); e.record(h2d_stream); ev_in.append(e)
            main_s.wait_event(ev_in[i])
            if use_graph:
                g_e2e[(k, sz)][0].replay()
                yk = g_e2e[(k, sz)][1]
            else:
                yk = forward(mconvs, x_chunk[k][:sz], sz, count=False)[0]
            lo_, hi_ = chunk_lo[i] * per_img_out, (chunk_lo[i] + sz) * per_img_out
            y_local[lo_:hi_].copy_(yk.reshape(-1), non_blocking=True)
            e = torch.cuda.Event(); e.record(main_s); ev_done.append(e)
            if world == 1:                               # single GPU: a chunk's result goes back while the next one computes
                with torch.cuda.stream(d2h_stream):
                    d2h_stream.wait_event(e)
                    y_host[lo_:hi_].copy_(y_local[lo_:hi_], non_blocking=True)
        if world == 1:
            main_s.wait_stream(d2h_stream)               # the step ends when the last result is on the host
            return y_local
        y = finish(y_local)
        if rank == 0:
            y_host.copy_(y, non_blocking=True)
        return y

    # ---- warm-up, then the timed regions ---------------------------------------------------------------
    for _ in range(max(args.warmup, 3)):
        step_value()
        step_e2e()
    barrier()
    uuid = str(torch.cuda.get_device_properties(dev).uuid)
    uuid = uuid if uuid.startswith("GPU-") else "GPU-" + uuid
    sampler = ClockSampler(uuid)
    sampler.start()
    time.sleep(0.15)
    barrier()
    ms_total = timed(step_value, args.steps)
    barrier()
    ms_total = max_over_ranks(ms_total)
    ms_nogather = None
    if world > 1:
        barrier()
        ms_nogather = max_over_ranks(timed(lambda: step_value(False), args.steps))
    barrier()
    ms_e2e = timed(step_e2e, args.steps)
    barrier()
    ms_e2e = max_over_ranks(ms_e2e)
    # the timed regions last a few milliseconds: keep the same steps running (untimed) until the sampler, which needs a
    # moment to start when several ranks query at once, has seen the GPU under this load
    t_load = time.time()
    while time.time() - t_load < 0.8:
        for _ in range(20):
            step_value(False)
        torch.cuda.synchronize()
    clocks = sampler.stop()
    gpu_launches = launches_per_step * args.steps

    # ---- sustained: back-to-back steps for >= sustained-seconds, no flush (each step moves > 4 GB at N = 1) ----------
    sustained = None
    if args.sustained_seconds > 0:
        per = ms_total / args.steps
        reps = max(int(args.sustained_seconds * 1e3 / max(per, 1e-3)), args.steps)
        s2 = ClockSampler(uuid)
        s2.start()
        barrier()
        ms_sus = max_over_ranks(timed(step_value, reps, flush=False))
        c2 = s2.stop()
        sustained = {"value": ops_per_step * reps / (ms_sus * 1e-3) / 1e12, "unit": "TOPS", "steps": reps, "seconds": ms_sus * 1e-3,
                     "ms_per_step": ms_sus / reps, "sm_mhz_median": c2["sm_mhz"], "power_w_max": c2.get("power_w_max"), "reasons": c2["reasons"],
                     "note": "steps back to back, no L2 flush between them (a step streams more than the L2 holds)"}

    # ---- parity: sampled images against the CPU oracle chain, outside every timed region ------------------------
    y_chk = step_value().clone()
    ths_in = tab_ops.residual_threshold(x_dev.reshape(n_local, -1), None, chain.THRESHOLD_SCALE)
    if world > 1:
        ths_all = torch.empty(N, dtype=torch.float32, device=dev)
        dist.all_gather_into_tensor(ths_all, ths_in)
    else:
        ths_all = ths_in
    y_e2e_chk = step_e2e().clone() if world == 1 else None
    torch.cuda.synchronize()
    parity = None
    if rank == 0:
        per_rank = N // world
        picks = sorted(set([0, N // 2, N - 1] + [r * per_rank + (r * 7) % max(per_rank, 1) for r in range(world)]))
        host_threads()
        yo = oracle_chain_images(x_host_full[picks].numpy(), ths_all[picks].cpu().numpy())
        got = y_chk.reshape(N, -1)[picks].cpu().numpy()
        ok = bool(np.array_equal(got, yo))
        if y_e2e_chk is not None:
            ok = ok and bool(np.array_equal(y_e2e_chk.reshape(N, -1)[picks].cpu().numpy(), yo))
        parity = {"images": len(picks), "image_indices": picks, "ok": ok,
                  "what": "final 7x7x512 outputs of the sampled images%s == CPU oracle chain on the GPU's input thresholds, bit for bit"
                          % (" (value and e2e paths)" if y_e2e_chk is not None else " (from the all-gathered tensor)")}
    del x_host_full

    if rank != 0:
        if world > 1:
            dist.barrier()
            dist.destroy_process_group()
        return

    value = ops_per_step * args.steps / (ms_total * 1e-3) / 1e12
    e2e_value = ops_per_step * args.steps / (ms_e2e * 1e-3) / 1e12
    stream = torch.cuda.current_stream(dev).cuda_stream

    def probe(kind):
        sink = torch.empty(lib.tab_pipe_probe_sink_bytes(), dtype=torch.uint8, device=dev)
        n_ops = ctypes.c_double(0)
        best = None
        for i in range(4):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            _cabi.check(lib.tab_pipe_probe_launch(kind, 4096 if kind < 5 else 1024, sink.data_ptr(), ctypes.byref(n_ops), stream), "probe")
            e1.record()
            torch.cuda.synchronize()
            ms = e0.elapsed_time(e1)
            if i > 0:
                best = ms if best is None else min(best, ms)
        return n_ops.value / (best * 1e-3)

    popc_rate = probe(0)          # lane-level POPC per second, whole device
    lop3_rate = probe(1)
    imma_sync_tops = probe(2) / 1e12   # s8 mma.sync from registers: the ceiling of the legacy MMA instruction
    umma_tops = probe(7) / 1e12        # tcgen05.mma kind::i8 128x256x32 from shared memory, no copies: the tensor ceiling
    # TNN per 32-bit word pair: 2 LOP3 to form t,u; f full adders (2 LOP3 each) per word and stream remove f POPC.
    # time(f) = max((2+4f)/lop3, 2(1-f)/popc); balanced f* gives the integer-pipe bound.
    f_star = min(max((2 * lop3_rate - 2 * popc_rate) / (4 * popc_rate + 2 * lop3_rate), 0.0), 1.0)
    pair_rate = 1.0 / max((2 + 4 * f_star) / lop3_rate, 2 * (1 - f_star) / popc_rate)
    peak_popc_tops = pair_rate * 64 / 1e12
    naive_popc_tops = popc_rate * 64 / 2 / 1e12

    try:
        peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
        bf16_peak, peak_src = float(peaks["bf16_tflops"]), "of measured"
        hbm_peak, hbm_src = float(peaks["hbm_gbs"]), "MEASURED_PEAKS.json hbm_gbs (of measured)"
    except Exception:
        bf16_peak, peak_src = 1590.0, "of fallback"
        hbm_peak, hbm_src = 6650.0, "fallback 6.65 TB/s (of fallback)"

    # ---- per-layer table: every launch of the step timed alone (CUDA events, L2 flushed) ---------------------------
    layer_rows = []
    sums = {"gemm_ms": 0.0, "popc_ms": 0.0, "quant_ms": 0.0, "ops": 0, "gemm_bytes": 0, "quant_bytes": 0}
    if not args.no_layer_table:
        h = H0
        jobs = []
        for b in chain.resnet18_blocks():
            oh_a = (h + 2 * b.conv_a.pad - b.conv_a.K + 1) // b.conv_a.stride
            jobs.append((b.conv_a, h, False))
            jobs.append((b.conv_b, oh_a, True))
            if b.shortcut is not None:
                jobs.append((b.shortcut, h, False))
            h = oh_a

        def time_launch(fn):
            times = []
            for i in range(6):
                flush_buf.fill_(1)
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                fn()
                e1.record()
                torch.cuda.synchronize()
                if i >= 2:
                    times.append(e0.elapsed_time(e1))
            return statistics.mean(times)

        state = tab_ops.new_state(n_local, dev)
        for cs, ih, has_res in jobs:
            oh = (ih + 2 * cs.pad - cs.K + 1) // cs.stride
            conv = convs[cs.name]
            xin = torch.randn(n_local, ih, ih, cs.C, device=dev)
            ths = tab_ops.residual_threshold(xin.reshape(n_local, -1), None, 0.7)
            qx = tab_ops.Quantize(xin, ths, 2, n_local, ih, ih, cs.C)[0]
            yb = torch.empty(n_local * oh * oh * cs.KN, dtype=torch.float32, device=dev)
            res = torch.round(torch.randn(n_local * oh * oh * cs.KN, device=dev) * 8) if has_res else None
            nxt = torch.empty(n_local, dtype=torch.float32, device=dev)
            btn = torch.empty(n_local, dtype=torch.int32, device=dev)
            geom = conv.geometry(n_local, ih, ih)
            chained = cs.K == 3                                             # the 3x3 convolutions feed thresholds, the shortcuts do not
            compact = chained and not has_res                               # a block's first convolution hands int16 to the next quantiser
            if compact:
                y16 = torch.empty(n_local * oh * oh * cs.KN, dtype=torch.int16, device=dev)
                ms_gemm = time_launch(lambda: _cabi.check(lib.tab_conv2d_bits_i16_launch(
                    qx.data_ptr(), conv.W8.data_ptr(), y16.data_ptr(), CONV_TYPE, *geom, state.data_ptr(), nxt.data_ptr(), 0.7, stream), "bits16"))
            else:
                ms_gemm = time_launch(lambda: _cabi.check(lib.tab_conv2d_bits_launch(
                    qx.data_ptr(), conv.W8.data_ptr(), yb.data_ptr(), CONV_TYPE, *geom, res.data_ptr() if has_res else None,
                    state.data_ptr() if chained else None, nxt.data_ptr() if chained else None, 0.7, stream), "bits"))
            kernel = lib.tab_last_conv_kernel().decode()
            if has_res:                                                     # a block's second convolution quantises the first one's int16 output
                x16 = torch.round(xin * 8).to(torch.int16)
                ms_quant = time_launch(lambda: _cabi.check(lib.tab_quantize_i16_launch(x16.data_ptr(), ths.data_ptr(), qx.data_ptr(), 2,
                                                                                        n_local, ih, ih, cs.C, stream), "quantize16"))
            else:
                ms_quant = time_launch(lambda: _cabi.check(lib.tab_quantize_launch(xin.data_ptr(), ths.data_ptr(), qx.data_ptr(), None, 2,
                                                                                    n_local, ih, ih, cs.C, stream), "quantize"))
            ms_popc = time_launch(lambda: _cabi.check(lib.tab_conv2d_packed_launch(qx.data_ptr(), conv.QW.data_ptr(), conv.BTN_W.data_ptr(), yb.data_ptr(),
                                                                                    CONV_TYPE, *geom, stream), "popc"))
            lops = 2 * n_local * oh * oh * cs.KN * cs.K * cs.K * cs.C
            gemm_bytes = qx.numel() * 8 + conv.W8.numel() + (2 * yb.numel() if compact else 4 * yb.numel() * (2 if has_res else 1))
            quant_bytes = (2 if has_res else 4) * xin.numel() + qx.numel() * 8
            sums["gemm_ms"] += ms_gemm; sums["popc_ms"] += ms_popc; sums["ops"] += lops; sums["gemm_bytes"] += gemm_bytes
            if cs.K == 3:                                                   # the shortcut reuses conv_a's bit-planes: no quantiser launch of its own
                sums["quant_ms"] += ms_quant; sums["quant_bytes"] += quant_bytes
            layer_rows.append({"layer": cs.name, "in": [ih, ih, cs.C], "KN": cs.KN, "K": cs.K, "s": cs.stride, "residual": has_res,
                               "gemm_kernel": kernel, "gemm_ms": round(ms_gemm, 4), "gemm_tops": round(lops / ms_gemm / 1e9, 1),
                               "gemm_GBps": round(gemm_bytes / ms_gemm / 1e6, 1),
                               "quantize_ms": round(ms_quant, 4), "quantize_GBps": round(quant_bytes / ms_quant / 1e6, 1),
                               "popcount_kernel_tops": round(lops / ms_popc / 1e9, 1)})
        assert lib.tab_device_status() == 0, "a bounded wait expired in the tensor-core kernel"

    # ---- TAB_Quantize alone at N=256, 56x56x256 (HBM-bound), against the measured copy bandwidth ---------
    quant = {}
    if world == 1:
        QN, QH, QW_, QC = 256, 56, 56, 256
        g2 = torch.Generator(device=dev)
        g2.manual_seed(1)
        xq = torch.randn(QN, QH, QW_, QC, device=dev, generator=g2)
        tq = (0.7 * xq.abs().mean(dim=(1, 2, 3))).contiguous()
        for bw in (2, 1):
            PC = QC // 64
            qx = torch.empty(QN * QH * QW_ * PC * bw, dtype=torch.int64, device=dev)
            btn = torch.empty(QN, dtype=torch.int32, device=dev)
            times = []
            for i in range(8):
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                _cabi.check(lib.tab_quantize_launch(xq.data_ptr(), tq.data_ptr(), qx.data_ptr(), btn.data_ptr(), bw, QN, QH, QW_, QC, stream), "quantize")
                e1.record()
                torch.cuda.synchronize()
                if i >= 3:
                    times.append(e0.elapsed_time(e1))
            ms = statistics.mean(times)
            nbytes = 4 * QN * QH * QW_ * QC + 4 * QN + 8 * QN * QH * QW_ * PC * bw + 4 * QN
            gbs = nbytes / ms / 1e6
            quant["bitwidth%d" % bw] = {"ms": round(ms, 4), "GBps": round(gbs, 1), "algorithmic_bytes": nbytes,
                                        "frac_of_measured_hbm": round(gbs / hbm_peak, 3)}
        quant.update({"metric": "TAB_Quantize HBM GB/s", "config": "N=256, 56x56x256 fp32 NHWC, input 822 MB > L2 (no flush needed)",
                      "peak_GBps": hbm_peak, "peak_source": hbm_src, "bound": "hbm"})
        del xq

    ms_step = ms_total / args.steps
    step_bytes = step_algorithmic_bytes(n_local)
    step_gbs = step_bytes / ms_step / 1e6
    gemm_achieved = sums["ops"] / (sums["gemm_ms"] * 1e-3) / 1e12 if sums["gemm_ms"] else None
    popc_achieved = sums["ops"] / (sums["popc_ms"] * 1e-3) / 1e12 if sums["popc_ms"] else None
    l1_images = n_local
    roofline = {
        "kernel": "whole step: %d launches (conv_umma_persist_kernel x19, quantize_auto_kernel x1 for the chain's input and its thresholds, quantize_c64_kernel x%d - the other convolutions' inputs are quantised by the kernel that wrote them)" % (launches_per_step, launches_per_step - 20),
        "bound": "hbm", "achieved": step_gbs, "peak": hbm_peak, "unit": "GB/s", "frac": step_gbs / hbm_peak, "peak_source": hbm_src,
        "algorithmic_bytes_per_step": step_bytes, "images_per_gpu": n_local,
        "traffic": (L1_TRAFFIC_PER_IMAGE * l1_images) if L1_TRAFFIC_PER_IMAGE else None,
        "traffic_note": "ncu dram bytes read + written of the step's largest launch (conv_umma_persist_kernel<2,64,6,1,2,1>, 56x56x64 -> 64 with "
                        "residual), captured at 64 images and scaled to this rank's %d images - a lower bound: at 64 images four fifths of the "
                        "output were still in the L2 when the launch ended; its algorithmic bytes are %.1fe6 (bit-planes + byte weights + fp32 "
                        "residual read + fp32 output)"
                        % (l1_images, (l1_images * 56 * 56 * 16 + 64 * 9 * 64 + 8 * l1_images * 56 * 56 * 64) / 1e6),
        "gemm_stage": {
            "kernel": "conv_umma_persist_kernel (persistent tcgen05.mma kind::i8 on bit-plane activations), %d launches per step, each timed alone" % len(layer_rows),
            "bound": "tensor", "achieved": gemm_achieved, "peak": umma_tops, "unit": "TOP/s",
            "frac": (gemm_achieved / umma_tops) if gemm_achieved else None,
            "frac_of_2x_bf16_measured": (gemm_achieved / (2.0 * bf16_peak)) if gemm_achieved else None,
            "hbm_GBps": (sums["gemm_bytes"] / (sums["gemm_ms"] * 1e-3) / 1e9) if sums["gemm_ms"] else None,
            "avg_launch_ms": sums["gemm_ms"] / max(len(layer_rows), 1),
            "peak_source": "measured in this run: tcgen05.mma kind::i8 128x256x32 issued back to back from shared memory on every SM (no copies, "
                           "no epilogue); 2 x MEASURED_PEAKS.json bf16_tflops would be %.0f TOP/s (%s); s8 mma.sync ceiling measured in this run: %.0f TOP/s"
                           % (2.0 * bf16_peak, peak_src, imma_sync_tops)},
        "quantize_in_step": {
            "kernel": "quantize_c64_kernel on the 16 convolution inputs of the step, each timed alone (inside the step 12 of them are launches of their own; the chain's input goes through quantize_auto_kernel, the small ones are quantised by the kernel that wrote them)", "bound": "hbm",
            "achieved": (sums["quant_bytes"] / (sums["quant_ms"] * 1e-3) / 1e9) if sums["quant_ms"] else None, "peak": hbm_peak, "unit": "GB/s"},
        "quantize": quant,
        "popcount": {
            "kernel": "conv_popc_kernel<TNN> (bit-packed LOP3/POPC path, TAB_PATH_POPCOUNT), same layers", "bound": "alu",
            "achieved": popc_achieved, "peak": peak_popc_tops, "unit": "TOP/s", "frac": (popc_achieved / peak_popc_tops) if popc_achieved else None,
            "peak_source": "measured in this run: POPC %.3e/s, LOP3 %.3e/s (register-only probe); balanced carry-save bound "
                           "(f*=%.2f full adders per word); one-POPC-per-word bound would be %.1f TOP/s" % (popc_rate, lop3_rate, f_star, naive_popc_tops)},
    }
    if roofline["quantize_in_step"]["achieved"]:
        roofline["quantize_in_step"]["frac"] = roofline["quantize_in_step"]["achieved"] / hbm_peak
    # the launch with the largest share of the step (two per step): the 56x56x64 -> 64 convolution with residual, HBM-bound
    dom = [r for r in layer_rows if r["layer"] in ("s1b0.b", "s1b1.b")]
    if dom:
        dom_ms = sum(r["gemm_ms"] for r in dom) / len(dom)
        dom_bytes = l1_images * 56 * 56 * 16 + 64 * 9 * 64 + 8 * l1_images * 56 * 56 * 64
        roofline["dominant_kernel"] = {
            "kernel": dom[0]["gemm_kernel"], "launches_per_step": len(dom), "bound": "hbm",
            "algorithmic_bytes_per_launch": dom_bytes, "avg_launch_ms": dom_ms,
            "achieved": dom_bytes / (dom_ms * 1e-3) / 1e9, "peak": hbm_peak, "unit": "GB/s",
            "frac": dom_bytes / (dom_ms * 1e-3) / 1e9 / hbm_peak,
            "traffic": (L1_TRAFFIC_PER_IMAGE * l1_images) if L1_TRAFFIC_PER_IMAGE else None,
            "note": "bit-planes and fp32 residual read, fp32 output written; timed alone with CUDA events, L2 flushed before the launch"}

    config = workload_config(world)
    config["parity_check"] = parity
    line = {
        "metric": "TAB_Conv2d binary-op TOPS", "value": value, "unit": "TOPS", "n_gpus": world, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": ms_step, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "s8 (ternary values on the integer tensor cores, s32 accumulate; exact)", "data": "synthetic",
        "config": config,
        "e2e": {"value": e2e_value, "unit": "TOPS", "ms_per_step": ms_e2e / args.steps,
                "h2d_bytes_per_step": int(x_host.numel() * 4), "d2h_bytes_per_step": int(N * per_img_out * 4),
                "api": "TAB_CUDA.Quantize / Conv2dBits (extension module, prepared weights) + pinned-host copies, %d chunks of images pipelined; bytes are rank 0's" % len(chunk_sizes)},
        "gpu_launches": gpu_launches, "launches_per_step": launches_per_step, "cuda_graph": bool(use_graph),
        "clocks": clocks,
        "roofline": roofline,
        "value_sustained": sustained,
        "layers": layer_rows,
    }
    if world > 1:
        line["value_no_gather"] = ops_per_step * args.steps / (ms_nogather * 1e-3) / 1e12
        line["ms_per_step_no_gather"] = ms_nogather / args.steps
    if world == 1 and not args.no_cpu_baseline:
        line["cpu_baseline"] = cpu_baseline(args.cpu_sample_images)
    emit(line)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    if parity is not None and not parity["ok"]:
        sys.stderr.write("parity check FAILED: sampled outputs differ from the CPU oracle\n")
        sys.exit(3)


if __name__ == "__main__":
    main()
