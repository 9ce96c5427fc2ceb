"""Benchmark of the embed + norm hot path on B200, next to candle's CPU path on the host cores.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload c1|c2|c3|c4|c5] [--impl reference]

One "step" is one pass of the hot path over one batch of synthetic token rows.  The default
workload is the largest single-GPU configuration and the one the row-sharded scaling target is
stated on: C5, RMSNorm + fused residual add, bf16, hidden 8192, 65536 token rows (3.2 GB of
compulsory HBM traffic per step).  Token rows are independent, so N GPUs each run the same number
of rows (weak scaling, no collective); the same 65536 rows split over the N GPUs (strong scaling)
are timed as well and reported under "strong_scaling".  C4 is the vocab-sharded exception, the one
configuration with an exchange step: at N >= 2 it is measured in the same run (all its variants)
and reported under "other_workloads.c4"; `--workload c4` makes it the headline.  At N = 1 the
other single-GPU configurations (C1, C2, C3 with both id orders) and the C5 row ladder (1 .. 8192
rows) are measured briefly in the same run and reported under "other_workloads".

Rank 0 prints ONE JSON line.  `value` is token rows per second with the inputs resident in HBM;
`e2e` is the same through the public front end with inputs coming from pinned host memory and the
normalised rows copied back to pinned host memory inside the timed region; `roofline` relates the
kernel's algorithmic bytes to the measured HBM copy bandwidth; `cpu_baseline` is the CPU oracle
(a restatement of candle's CPU code, threaded the way candle threads it) on a bounded sample.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

import numpy as np  # noqa: E402

SEED = 0
L2_BYTES = 126 * 1024 * 1024
METRIC = "tokens/s, embed+norm (HBM GB/s in roofline)"

# dram__bytes_read.sum + dram__bytes_write.sum per launch of the dominant kernel, from the ncu
# captures summarised under profiles/ (the part of the output still dirty in L2 when the kernel ends
# is not in these figures; each summary says how much that is).  c5: 268.5 MB read and 96.0 MB
# written on the 8192-row capture; reads and writes grow with the rows, the ~38 MB left in L2 do not:
# 8 x 268.5 + 8 x 134.2 - 38 MB.
NCU_TRAFFIC_BYTES = {"c1": 87_100_000, "c2": 51_600_000, "c3": 540_400_000, "c5": 3_184_000_000, "c4": None}


def measured_peak():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


def host_cores() -> int:
    """The cores this process may run on, whatever OMP_NUM_THREADS says (torchrun sets it to 1);
    candle's rayon pool sizes itself the same way."""
    try:
        return max(1, len(os.sched_getaffinity(0)))
    except AttributeError:
        return os.cpu_count() or 1


# ------------------------------------------------------------------------------------------------
# workloads: seeded synthetic inputs with the shapes and value distributions of the configs
# ------------------------------------------------------------------------------------------------
def zipf_ids(rng, vocab, n, s=1.1):
    p = 1.0 / np.arange(1, vocab + 1, dtype=np.float64) ** s
    p /= p.sum()
    return rng.choice(vocab, size=n, p=p).astype(np.uint32)  # rank k -> id k-1


class Workload:
    """Holds host-side inputs (numpy, oracle layout) and knows its algorithmic bytes per step."""

    def __init__(self, name, rows_scale=1.0, permuted=False):
        from helpers import make_qtable, randn

        rng = np.random.default_rng(SEED)
        self.name = name
        if name == "c1":
            self.desc = "C1 Llama embed+RMSNorm f32: table 32000x4096 N(0,0.02), ids uniform 8x512, eps 1e-5"
            self.vocab, self.hidden, self.rows, self.dtype = 32000, 4096, 8 * 512, "f32"
            self.table = randn(rng, (self.vocab, self.hidden), "f32", 0.0, 0.02)
            self.alpha = randn(rng, (self.hidden,), "f32", 1.0, 0.1)
            self.n_sets = 4  # 134 MB per step is close to L2: rotate over 4 id/output sets
            self.ids = [rng.integers(0, self.vocab, size=self.rows).astype(np.uint32) for _ in range(self.n_sets)]
            self.bytes_per_step = self.rows * self.hidden * 4 * 2
            self.eps = 1e-5
        elif name == "c2":
            self.desc = "C2 BERT LayerNorm bf16 + residual: x,res 16384x768 N(0,1), eps 1e-12"
            self.rows, self.hidden, self.dtype = 16384, 768, "bf16"
            self.n_sets = 12  # 75 MB per step fits L2: rotate over 12 buffer sets (> 2x L2 in total)
            self.x = [randn(rng, (self.rows, self.hidden), "bf16") for _ in range(2)]
            self.res = [randn(rng, (self.rows, self.hidden), "bf16") for _ in range(2)]
            self.gamma = randn(rng, (self.hidden,), "bf16", 1.0, 0.1)
            self.beta = randn(rng, (self.hidden,), "bf16", 0.0, 0.1)
            self.bytes_per_step = 3 * self.rows * self.hidden * 2
            self.eps = 1e-12
        elif name in ("c3", "c4"):
            if name == "c3":
                order = ("a seeded permutation of the vocabulary (hot rows scattered over the table)" if permuted
                         else "rank k -> id k-1 (hot rows contiguous at the table start)")
                self.desc = f"C3 GGUF Q8_0 embedding 128256x4096 -> bf16 -> RMSNorm eps 1e-5, ids Zipf(1.1) 32x2048, {order}"
                self.vocab, self.hidden, self.rows, self.qtype = 128256, 4096, 32 * 2048, "q8_0"
            else:
                self.desc = ("C4 GGUF Q4_0 embedding 152064x8192 vocab-sharded, ids uniform 64x4096, lookup + exchange "
                             "over NVLink + RMSNorm eps 1e-5")
                self.vocab, self.hidden, self.rows, self.qtype = 152064, 8192, int(64 * 4096 * rows_scale), "q4_0"
            self.dtype = "bf16"
            self.qtable = make_qtable(rng, self.qtype, self.vocab, self.hidden)
            self.alpha = randn(rng, (self.hidden,), "bf16", 1.0, 0.1)
            self.n_sets = 2
            gen = (lambda: zipf_ids(rng, self.vocab, self.rows)) if name == "c3" else (
                lambda: rng.integers(0, self.vocab, size=self.rows).astype(np.uint32))
            self.ids = [gen() for _ in range(self.n_sets)]
            if permuted:
                perm = rng.permutation(self.vocab).astype(np.uint32)
                self.ids = [perm[i] for i in self.ids]
            self.row_qbytes = self.qtable.shape[1]
            self.bytes_per_step = self.rows * (self.row_qbytes + self.hidden * 2)
            self.eps = 1e-5
        elif name == "c5":
            self.rows = max(1, int(round(65536 * rows_scale)))
            self.desc = f"C5 RMSNorm + residual bf16, hidden 8192, {self.rows} token rows, eps 1e-5"
            self.hidden, self.dtype = 8192, "bf16"
            self.bytes_per_step = 3 * self.rows * self.hidden * 2
            # cold-L2 protocol: one set if a step alone is several times L2, else enough sets for 2x L2
            self.n_sets = 1 if self.bytes_per_step > 4 * L2_BYTES else int(min(64, max(8, -(-2 * L2_BYTES // self.bytes_per_step))))
            base = min(self.rows, 4096)  # seeded block, tiled to the full row count
            self.x = [randn(rng, (base, self.hidden), "bf16") for _ in range(1)]
            self.res = [randn(rng, (base, self.hidden), "bf16") for _ in range(1)]
            self.alpha = randn(rng, (self.hidden,), "bf16", 1.0, 0.1)
            self.eps = 1e-5
        else:
            raise SystemExit(f"unknown workload {name}")

    def l2_note(self):
        return (f"rotating {self.n_sets} buffer set(s); working set per step {self.bytes_per_step / 1e6:.1f} MB "
                f"vs 126 MB L2")


def config_of(wl, world, parallelism=None):
    """The `config` object, identical in the GPU arm and the reference arm."""
    return {"workload": wl.desc, "rows_per_gpu": wl.rows, "hidden": wl.hidden,
            "parallelism": parallelism or f"token rows x{world}, no collective", "l2": wl.l2_note()}


def parity_sample(rows, hidden=0, limit=4096, stride=17):
    """Row numbers the full-size parity check compares: every row while the oracle takes well under a
    second (up to 2^26 elements), else every 17th row up to `limit` rows (17 is coprime to the 4096-row
    seeded block the dense inputs are tiled from)."""
    if rows <= limit or rows * hidden <= (1 << 26):
        return np.arange(rows)
    return np.arange(0, rows, stride)[:limit]


# ------------------------------------------------------------------------------------------------
# GPU arm
# ------------------------------------------------------------------------------------------------
class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons while the timed region runs."""

    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.lines, self.proc = index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "100", "-i", str(self.index)],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._pump, daemon=True).start()
        except OSError:
            self.proc = None

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        sm, mx, reasons = [], [], set()
        for l in self.lines:
            f = [p.strip() for p in l.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                mx.append(float(f[2]))
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


class Runner:
    """Device-resident inputs of one workload plus the closures that launch it and check it."""

    def __init__(self, wl, dev, stream, st, e2e=True):
        import torch

        import candle_b200 as cb
        from candle_b200 import _cabi
        from helpers import from_oracle, ids_tensor, to_oracle
        import oracle

        self.wl, S = wl, wl.n_sets
        self.e2e_step = None
        sample = parity_sample(wl.rows, wl.hidden)
        self.parity_rows = len(sample)
        if wl.name in ("c1", "c3"):
            if wl.name == "c1":
                table = from_oracle(wl.table, wl.dtype, dev)
                out_dt = table.dtype
            else:
                q = cb.QTensor.from_raw(torch.from_numpy(wl.qtable), cb.GgmlDType.Q8_0, (wl.vocab, wl.hidden), device=dev)
                out_dt = torch.bfloat16
            alpha = from_oracle(wl.alpha, wl.dtype, dev)
            ids = [ids_tensor(i, dev) for i in wl.ids]
            ys = [torch.empty(wl.rows, wl.hidden, dtype=out_dt, device=dev) for _ in range(S)]

            if wl.name == "c1":
                def launch(ids_ptr, y):
                    _cabi.call("cb200_embedding_rms_norm", table.data_ptr(), ids_ptr, alpha.data_ptr(), y.data_ptr(), None,
                               wl.vocab, wl.hidden, wl.rows, wl.eps, 0, 1, 0, st.data_ptr(), stream.cuda_stream)

                def want():
                    return oracle.rms_norm(oracle.embedding(wl.table, wl.ids[0][sample]), wl.alpha, wl.eps, "f32")
            else:
                def launch(ids_ptr, y):
                    _cabi.call("cb200_qembedding_rms_norm", q.data.data_ptr(), q.dtype.value, ids_ptr, alpha.data_ptr(),
                               y.data_ptr(), None, wl.vocab, wl.hidden, wl.rows, wl.eps, 2, 1, 0, wl.vocab, 0,
                               st.data_ptr(), stream.cuda_stream)

                def want():
                    return oracle.rms_norm(oracle.qembedding(wl.qtable, wl.qtype, wl.ids[0][sample], "bf16"), wl.alpha,
                                           wl.eps, "bf16")

            self.step = lambda i: launch(ids[i % S].data_ptr(), ys[i % S])
            idx = torch.from_numpy(sample).to(dev)
            self.check = lambda: np.array_equal(to_oracle(ys[0][idx]), want())
            if e2e:
                host_in = [torch.from_numpy(i.view(np.int32)).pin_memory() for i in wl.ids]
                dev_in = torch.empty(wl.rows, dtype=torch.int32, device=dev)

                def e2e_step(i, host_out):
                    dev_in.copy_(host_in[i % S], non_blocking=True)
                    launch(dev_in.data_ptr(), ys[0])
                    host_out.copy_(ys[0], non_blocking=True)
                self.e2e_step = e2e_step
            self.h2d = wl.rows * 4
        else:  # c2 / c5: dense rows + residual
            base = wl.x[0].shape[0]
            reps = -(-wl.rows // base)
            xs, rs, ys = [], [], []
            for s in range(S):
                bx = from_oracle(wl.x[s % len(wl.x)], "bf16", dev)
                br = from_oracle(wl.res[s % len(wl.res)], "bf16", dev)
                xs.append(bx.repeat(reps, 1)[: wl.rows].contiguous())
                rs.append(br.repeat(reps, 1)[: wl.rows].contiguous())
                ys.append(torch.empty(wl.rows, wl.hidden, dtype=torch.bfloat16, device=dev))
            h = oracle.add(wl.x[0][sample % base], wl.res[0][sample % base], "bf16")
            idx = torch.from_numpy(sample).to(dev)
            if wl.name == "c2":
                g, b = from_oracle(wl.gamma, "bf16", dev), from_oracle(wl.beta, "bf16", dev)

                def launch(x, r, y):
                    _cabi.call("cb200_layer_norm", x.data_ptr(), r.data_ptr(), g.data_ptr(), b.data_ptr(), y.data_ptr(),
                               None, wl.rows, wl.hidden, wl.eps, 2, 0, stream.cuda_stream)
                self.check = lambda: np.array_equal(
                    to_oracle(ys[0][idx]), oracle.layer_norm(h, wl.gamma, wl.beta, wl.eps, "bf16"))
            else:
                a = from_oracle(wl.alpha, "bf16", dev)

                def launch(x, r, y):
                    _cabi.call("cb200_rms_norm", x.data_ptr(), r.data_ptr(), a.data_ptr(), y.data_ptr(), None, wl.rows,
                               wl.hidden, wl.eps, 2, 0, stream.cuda_stream)
                self.check = lambda: np.array_equal(to_oracle(ys[0][idx]), oracle.rms_norm(h, wl.alpha, wl.eps, "bf16"))
            self.step = lambda i: launch(xs[i % S], rs[i % S], ys[i % S])
            if e2e:
                host_x, host_r = xs[0].cpu().pin_memory(), rs[0].cpu().pin_memory()
                # end to end through the library's pinned-host front end: rows in chunks, copy in / kernel /
                # copy out overlapped on three streams
                chunk = max(1024, wl.rows // 8)
                pipe = cb.PinnedNormPipeline(wl.hidden, torch.bfloat16, dev, chunk_rows=chunk)
                self.e2e_note = f"PinnedNormPipeline, chunks of {pipe.chunk_rows} rows on three streams"

                def e2e_step(i, host_out):
                    if wl.name == "c2":
                        pipe.run(host_x, host_out, g, wl.eps, residual_host=host_r, beta=b)
                    else:
                        pipe.run(host_x, host_out, a, wl.eps, residual_host=host_r)
                self.e2e_step = e2e_step

                # the same bytes with no kernel in between: one cudaMemcpyAsync per chunk each way,
                # both directions at once -- what the host link alone allows
                dx = [torch.empty(chunk, wl.hidden, dtype=torch.bfloat16, device=dev) for _ in range(2)]
                s_in, s_out = torch.cuda.Stream(dev), torch.cuda.Stream(dev)

                def copy_only(i, host_out):
                    cur = torch.cuda.current_stream(dev)
                    s_in.wait_stream(cur)
                    s_out.wait_stream(cur)
                    for begin in range(0, wl.rows, chunk):
                        n = min(chunk, wl.rows - begin)
                        with torch.cuda.stream(s_in):
                            dx[0][:n].copy_(host_x[begin:begin + n], non_blocking=True)
                            dx[0][:n].copy_(host_r[begin:begin + n], non_blocking=True)
                        with torch.cuda.stream(s_out):
                            host_out[begin:begin + n].copy_(dx[1][:n], non_blocking=True)
                    cur.wait_stream(s_in)
                    cur.wait_stream(s_out)
                self.copy_only = copy_only
            self.h2d = 2 * wl.rows * wl.hidden * 2
        self.out_dtype = ys[0].dtype


class Timer:
    """CUDA-event timing on the launching stream, bracketed by barrier + synchronize, max over ranks."""

    def __init__(self, dev, world):
        import torch
        import torch.distributed as dist

        self.torch, self.dist, self.dev, self.world = torch, dist, dev, world
        self.stream = torch.cuda.current_stream()

    def barrier(self):
        if self.world > 1:
            self.dist.barrier()
        self.torch.cuda.synchronize()

    def __call__(self, fn, steps, warmup):
        torch = self.torch
        for i in range(warmup):
            fn(i)
        self.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(self.stream)
        for i in range(steps):
            fn(warmup + i)
        e1.record(self.stream)
        self.barrier()
        ms = e0.elapsed_time(e1)
        if self.world > 1:
            t = torch.tensor([ms], device=self.dev)
            self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
            ms = t.item()
        return ms


def brief_workload(name, dev, stream, st, timed, peak, **kw):
    """One of the other configurations, measured briefly: parity first, then 20 launches."""
    import torch

    w = Workload(name, **kw)
    if w.bytes_per_step < 8e6:
        # a call this small is shorter than the host's launch path: time the device with a CUDA graph of
        # back-to-back launches (rotating buffer sets), so that what is reported is not the host
        side = torch.cuda.Stream(dev)
        side.wait_stream(torch.cuda.current_stream(dev))
        r = Runner(w, dev, side, st, e2e=False)
        with torch.cuda.stream(side):
            for i in range(5):
                r.step(i)
        torch.cuda.synchronize()
        ok = bool(r.check())
        n_cap = max(w.n_sets, 32)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):
            for i in range(n_cap):
                r.step(i)
        torch.cuda.synchronize()
        ms = timed(lambda i: graph.replay(), 10, 3) / (10 * n_cap)
        how = f"device time per launch inside a CUDA graph of {n_cap} back-to-back launches"
    else:
        r = Runner(w, dev, stream, st, e2e=False)
        r.step(0)
        torch.cuda.synchronize()
        ok = bool(r.check())
        k = 20
        ms = timed(r.step, k, 5) / k
        how = f"CUDA events around {k} back-to-back launches"
    gbs = w.bytes_per_step / (ms * 1e-3) / 1e9
    out = {"workload": w.desc, "rows": w.rows, "ms_per_step": ms, "us_per_step": ms * 1e3,
           "tokens_per_s": w.rows / (ms * 1e-3), "achieved_gbs": gbs, "frac_of_measured_peak": gbs / peak,
           "algorithmic_bytes_per_launch": w.bytes_per_step, "l2": w.l2_note(), "timing": how,
           "parity": f"bit-exact vs CPU oracle on {r.parity_rows} of {w.rows} rows" if ok else "MISMATCH",
           "ncu_traffic_bytes": NCU_TRAFFIC_BYTES.get(name) if not kw else None}
    del r, w
    torch.cuda.empty_cache()
    return out, ok


def next_rows_section(dev, timed, peak):
    """The operators next to the hot path (composite norm, softmax, rope, K-quant lookups, the norm
    of selected rows), each briefly: parity against the oracle on rows of these very inputs, then 10
    launches on inputs larger than L2."""
    import torch

    import oracle
    from candle_b200 import ops
    from candle_b200.quantized import GgmlDType, QTensor
    from helpers import from_oracle, ids_tensor, make_kq_blocks, randn, to_oracle

    rng = np.random.default_rng(SEED + 1)
    out, all_ok = {}, True

    def entry(name, desc, fn, nbytes, ok, how):
        nonlocal all_ok
        k = 10
        ms = timed(lambda i: fn(), k, 3) / k
        gbs = nbytes / (ms * 1e-3) / 1e9
        out[name] = {"workload": desc, "us_per_step": ms * 1e3, "achieved_gbs": gbs, "frac_of_measured_peak": gbs / peak,
                     "algorithmic_bytes_per_launch": nbytes, "parity": how if ok else "MISMATCH"}
        all_ok = all_ok and ok
        torch.cuda.empty_cache()

    def tiled(block, reps):  # a seeded block repeated: parity is checked on the first block
        return from_oracle(block, "bf16", dev).repeat(reps, 1)

    # ---- candle's composite norm chain (layer_norm.rs:108-136), bf16 ----
    rows, hidden, base = 65536, 4096, 512
    xb = randn(rng, (base, hidden), "bf16")
    w, b = randn(rng, (hidden,), "bf16", 1.0, 0.1), randn(rng, (hidden,), "bf16", 0.0, 0.1)
    x, tw, tb = tiled(xb, rows // base), from_oracle(w, "bf16", dev), from_oracle(b, "bf16", dev)
    for name, bias, rm in (("rms_norm_slow", None, False), ("layer_norm_slow", b, True)):
        f = (lambda: ops.rms_norm_slow(x, tw, 1e-5)) if bias is None else (lambda: ops.layer_norm_slow(x, tw, tb, 1e-5))
        ok = np.array_equal(to_oracle(f()[:base]), oracle.norm_slow(xb, w, bias, 1e-5, "bf16", remove_mean=rm))
        entry(name, f"candle's composite norm chain, bf16, {rows} x {hidden}", f, 2 * rows * hidden * 2, ok,
              f"bit-exact vs CPU oracle on {base} rows")
    del x
    # ---- softmax over the last dimension ----
    rows, n, base = 65536, 2048, 256
    for dt in ("f32", "bf16"):
        xb = randn(rng, (base, n), dt, 0.0, 3.0)
        x = from_oracle(xb, dt, dev).repeat(rows // base, 1)
        got = oracle.cast_to_f32(to_oracle(ops.softmax_last_dim(x)[:base]), dt)
        want = oracle.cast_to_f32(oracle.softmax_last_dim(xb, dt), dt)
        tol = 1e-5 if dt == "f32" else 1e-2
        es = 4 if dt == "f32" else 2
        entry(f"softmax_last_dim_{dt}", f"softmax over the last dimension, {dt}, {rows} x {n}",
              lambda: ops.softmax_last_dim(x), 2 * rows * n * es, bool(np.abs(got - want).max() <= tol),
              f"max |diff| {float(np.abs(got - want).max()):.2e} <= {tol} vs CPU oracle on {base} rows (exp from two math libraries)")
        del x
    # ---- rotary embeddings ----
    bsz, h, t, d = 8, 32, 2048, 128
    cos, sin = randn(rng, (t, d // 2), "bf16"), randn(rng, (t, d // 2), "bf16")
    tc, ts = from_oracle(cos, "bf16", dev), from_oracle(sin, "bf16", dev)
    for variant in ("rope_i", "rope", "rope_thd"):
        shape1 = (1, t, h, d) if variant == "rope_thd" else (1, h, t, d)
        xb = randn(rng, shape1, "bf16")
        x = from_oracle(xb, "bf16", dev).repeat(bsz, 1, 1, 1)
        f = getattr(ops, variant)
        ok = np.array_equal(to_oracle(f(x, tc, ts)[:1]), oracle.rope(variant, xb, cos, sin, "bf16"))
        entry(variant, f"{variant}, bf16, b {bsz} h {h} t {t} d {d}", lambda: f(x, tc, ts), 2 * x.numel() * 2, ok,
              "bit-exact vs CPU oracle on one batch element")
        del x
    # ---- lookups from K-quant tables ----
    vocab, hidden, n_ids, sample = 8192, 4096, 65536, 512
    ids = rng.integers(0, vocab, size=n_ids).astype(np.uint32)
    tids = ids_tensor(ids, dev)
    alpha = randn(rng, (hidden,), "bf16", 1.0, 0.1)
    ta = from_oracle(alpha, "bf16", dev)
    for qname in ("q4k", "q6k"):
        gq = getattr(GgmlDType, qname.upper())
        raw = make_kq_blocks(rng, qname, vocab * hidden // 256).reshape(vocab, -1)
        q = QTensor.from_raw(torch.from_numpy(raw), gq, (vocab, hidden), device=dev)
        rows_q = oracle.qembedding(raw, qname, ids[:sample], "bf16")
        ok = np.array_equal(to_oracle(q.embedding(tids, torch.bfloat16)[:sample]), rows_q)
        entry(f"qembedding_{qname}", f"lookup from a {qname.upper()} table {vocab} x {hidden} -> bf16, {n_ids} ids",
              lambda: q.embedding(tids, torch.bfloat16, check=False), n_ids * (raw.shape[1] + hidden * 2), ok,
              f"bit-exact vs CPU oracle on {sample} rows")
        ok = np.array_equal(to_oracle(ops.qembedding_rms_norm(q, tids, ta, 1e-5)[:sample]),
                            oracle.rms_norm(rows_q, alpha, 1e-5, "bf16"))
        entry(f"qembedding_rms_norm_{qname}", "the same lookup + RMS norm, one launch",
              lambda: ops.qembedding_rms_norm(q, tids, ta, 1e-5, check=False), n_ids * (raw.shape[1] + hidden * 2), ok,
              f"bit-exact vs CPU oracle on {sample} rows")
        del q
    # ---- the norm of selected rows (the final norm feeds one token per sequence into the LM head) ----
    rows, hidden, picks = 16384, 8192, 64
    xb = randn(rng, (512, hidden), "bf16")
    x = tiled(xb, rows // 512)
    alpha = randn(rng, (hidden,), "bf16", 1.0, 0.1)
    ta = from_oracle(alpha, "bf16", dev)
    sel = np.sort(rng.choice(rows, size=picks, replace=False)).astype(np.int64)
    tsel = torch.from_numpy(sel).to(dev)
    ok = np.array_equal(to_oracle(ops.rms_norm_rows(x, tsel, ta, 1e-5)), oracle.rms_norm(xb[sel % 512], alpha, 1e-5, "bf16"))
    # a call this small is shorter than the host's launch path: device time inside a CUDA graph
    from candle_b200 import _cabi

    side = torch.cuda.Stream(dev)
    side.wait_stream(torch.cuda.current_stream(dev))
    ysel = torch.empty(picks, hidden, dtype=torch.bfloat16, device=dev)
    st = ops.new_status(dev)

    def launch():
        _cabi.call("cb200_embedding_rms_norm", x.data_ptr(), tsel.data_ptr(), ta.data_ptr(), ysel.data_ptr(), None, rows,
                   hidden, picks, 1e-5, 2, 2, 0, st.data_ptr(), side.cuda_stream)

    with torch.cuda.stream(side):
        for _ in range(3):
            launch()
    torch.cuda.synchronize()
    n_cap = 32
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=side):
        for _ in range(n_cap):
            launch()
    torch.cuda.synchronize()
    ms_sel = timed(lambda i: graph.replay(), 10, 3) / (10 * n_cap)
    k = 20
    ms_all = timed(lambda i: ops.rms_norm(x, ta, 1e-5), k, 3) / k
    out["rms_norm_selected_rows"] = {
        "workload": f"RMS norm bf16 of {picks} selected rows of {rows} x {hidden} (candle norms all rows, then slices)",
        "us_per_step": ms_sel * 1e3, "us_per_step_all_rows": ms_all * 1e3,
        "timing": f"device time per launch inside a CUDA graph of {n_cap} back-to-back launches",
        "parity": f"bit-exact vs CPU oracle on the {picks} rows" if ok else "MISMATCH"}
    all_ok = all_ok and ok
    return out, all_ok


def gpu_arm(args):
    import torch
    import torch.distributed as dist

    from candle_b200.ops import new_status, raise_for_status

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torch.distributed.run for N > 1")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
        dist.init_process_group("nccl", device_id=dev)
    timed = Timer(dev, world)
    peak, peak_kind = measured_peak()
    if args.workload == "next":
        if world != 1:
            raise SystemExit("--workload next runs on one GPU")
        out, ok = next_rows_section(dev, timed, peak)
        print(json.dumps({"next_rows": out}), flush=True)
        if not ok:
            raise SystemExit(3)
        return
    if args.workload == "c4":
        if world < 2:
            raise SystemExit("the vocab-sharded C4 workload needs --gpus >= 2 (launch with torch.distributed.run)")
        c4, ok = c4_section(args, rank, world, dev, timed, peak, headline=True)
        if rank == 0:
            print(json.dumps(c4), flush=True)
        dist.destroy_process_group()
        if not ok:
            raise SystemExit(3)
        return

    stream = timed.stream
    st = new_status(dev)
    wl = Workload(args.workload, args.rows_scale)
    run = Runner(wl, dev, stream, st)

    # ---- parity on this very workload before anything is timed ----
    run.step(0)
    torch.cuda.synchronize()
    raise_for_status(st)
    parity_ok = bool(run.check())

    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    ms = timed(run.step, args.steps, args.warmup)
    if rank == 0:
        # the timed region can be shorter than one nvidia-smi sampling period: keep the same launches going
        # (untimed) for 0.4 s so that the clock record has samples taken under this load
        t_end, i = time.time() + 0.4, 0
        while time.time() < t_end:
            run.step(i)
            i += 1
            if i % 32 == 0:
                torch.cuda.synchronize()
        torch.cuda.synchronize()
    clocks = sampler.stop() if rank == 0 else None
    if clocks is not None:
        clocks["window"] = "timed region + 0.4 s of the same launches, 100 ms period"
    timed.barrier()
    raise_for_status(st)

    # ---- end to end: host buffers in, host rows out, through the same call ----
    host_out = torch.empty(wl.rows, wl.hidden, dtype=run.out_dtype).pin_memory()
    e2e_steps = max(2, min(args.steps, 10))
    e2e_ms = timed(lambda i: run.e2e_step(i, host_out), e2e_steps, 1)
    d2h = host_out.numel() * host_out.element_size()
    e2e_how = getattr(run, "e2e_note", "one call per step: ids from pinned host memory in, rows to pinned host memory out")
    copy_ms = None
    if hasattr(run, "copy_only"):
        copy_ms = timed(lambda i: run.copy_only(i, host_out), e2e_steps, 1)

    others = {}
    if not args.no_sweep:
        del run, host_out
        torch.cuda.empty_cache()
        if world == 1:
            for name in ("c1", "c2", "c3", "c5"):
                if name == wl.name:
                    continue
                others[name], ok2 = brief_workload(name, dev, stream, st, timed, peak)
                parity_ok = parity_ok and ok2
            others["c3_permuted_ids"], ok2 = brief_workload("c3", dev, stream, st, timed, peak, permuted=True)
            parity_ok = parity_ok and ok2
            ladder = {}
            for rows in (1, 8, 64, 512, 8192):
                ladder[str(rows)], ok2 = brief_workload("c5", dev, stream, st, timed, peak, rows_scale=rows / 65536)
                parity_ok = parity_ok and ok2
            others["c5_rows"] = ladder
            others["next_rows"], ok2 = next_rows_section(dev, timed, peak)
            parity_ok = parity_ok and ok2
        else:
            if wl.name == "c5" and args.rows_scale == 1.0:
                # strong scaling: the 65536 rows of the configuration split over the ranks
                w2 = Workload("c5", 1.0 / world)
                r2 = Runner(w2, dev, stream, st, e2e=False)
                r2.step(0)
                torch.cuda.synchronize()
                ok2 = bool(r2.check())
                k = 50
                ms2 = timed(r2.step, k, 5) / k
                gbs = w2.bytes_per_step / (ms2 * 1e-3) / 1e9
                others["strong_scaling"] = {
                    "workload": f"C5, 65536 token rows split over {world} GPUs ({w2.rows} rows each), no collective",
                    "scaling": "strong", "ms_per_step": ms2, "tokens_per_s": world * w2.rows / (ms2 * 1e-3),
                    "achieved_gbs_per_gpu": gbs, "frac_of_measured_peak": gbs / peak, "l2": w2.l2_note(),
                    "parity": f"bit-exact vs CPU oracle on {r2.parity_rows} rows per rank" if ok2 else "MISMATCH"}
                parity_ok = parity_ok and ok2
                del r2, w2
                torch.cuda.empty_cache()
            c4, ok2 = c4_section(args, rank, world, dev, timed, peak, headline=False)
            others["c4"] = c4
            parity_ok = parity_ok and ok2
    if world > 1:
        flag = torch.tensor([1.0 if parity_ok else 0.0], device=dev)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        parity_ok = bool(flag.item() == 1.0)

    if rank == 0:
        ms_per_step = ms / args.steps
        achieved = wl.bytes_per_step / (ms_per_step * 1e-3) / 1e9
        e2e_value = world * wl.rows * e2e_steps / (e2e_ms * 1e-3)
        e2e = {"value": e2e_value, "unit": "tokens/s", "h2d_bytes_per_step": run_h2d(wl), "d2h_bytes_per_step": d2h,
               "ms_per_step": e2e_ms / e2e_steps, "how": e2e_how}
        if copy_ms is not None:
            ceiling = world * wl.rows * e2e_steps / (copy_ms * 1e-3)
            e2e.update({"copy_ceiling_tokens_per_s": ceiling, "frac_of_copy_ceiling": e2e_value / ceiling,
                        "copy_ceiling_how": "the same host->device and device->host bytes on the same ranks, one "
                                            "cudaMemcpyAsync per chunk each way on two streams, no kernel",
                        "host_link_gbs_per_rank": (run_h2d(wl) + d2h) / (copy_ms / e2e_steps * 1e-3) / 1e9})
        out = {
            "metric": METRIC,
            "value": world * wl.rows * args.steps / (ms * 1e-3),
            "unit": "tokens/s",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_per_step,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": wl.dtype, "data": "synthetic (seed 0)",
            "config": config_of(wl, world),
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                         "peak_kind": f"of {peak_kind}", "frac_of_nominal_8000": achieved / 8000.0,
                         "algorithmic_bytes_per_launch": wl.bytes_per_step,
                         "traffic": NCU_TRAFFIC_BYTES.get(wl.name) if args.rows_scale == 1.0 else None},
            "e2e": e2e,
            "gpu_launches": args.steps,
            "parity": (f"bit-exact vs CPU oracle on {len(parity_sample(wl.rows, wl.hidden))} of {wl.rows} rows"
                       if parity_ok else "MISMATCH vs CPU oracle"),
            "clocks": clocks,
        }
        if others:
            out["other_workloads"] = others
        if not args.no_cpu and world == 1:
            out["cpu_baseline"] = cpu_baseline(wl)
        print(json.dumps(out), flush=True)
    if world > 1:
        dist.destroy_process_group()
    if not parity_ok:
        raise SystemExit(3)


def run_h2d(wl):
    return wl.rows * 4 if wl.name in ("c1", "c3") else 2 * wl.rows * wl.hidden * 2


# ------------------------------------------------------------------------------------------------
# C4: the vocabulary-sharded table, the one configuration with an exchange between GPUs
# ------------------------------------------------------------------------------------------------
def c4_section(args, rank, world, dev, timed, peak, headline):
    """All variants of the vocab-sharded lookup + RMS norm on `world` GPUs.  Returns (dict, parity_ok);
    with `headline` the dict is a complete bench line (fastest variant), else an `other_workloads` entry."""
    import torch
    import torch.distributed as dist

    from candle_b200 import ops
    from candle_b200.parallel import (RoutedQEmbedding, ShardedQEmbedding, as_words, peer_mapped_empty, row_shard,
                                      vocab_shard)
    from candle_b200.quantized import GgmlDType, QTensor
    from helpers import from_oracle, ids_tensor, to_oracle
    import oracle

    wl = Workload("c4", args.rows_scale if headline else 1.0)
    steps = args.steps if headline else 6
    begin, end = vocab_shard(wl.vocab, rank, world)
    local = QTensor.from_raw(torch.from_numpy(wl.qtable[begin:end]), GgmlDType.Q4_0, (end - begin, wl.hidden), device=dev)
    emb = ShardedQEmbedding(local, wl.vocab, rank, world, torch.bfloat16)
    alpha = from_oracle(wl.alpha, "bf16", dev)
    ids = [ids_tensor(i, dev) for i in wl.ids]
    st = ops.new_status(dev)
    out_bytes = wl.rows * wl.hidden * 2
    rb, re = row_shard(wl.rows, rank, world)

    # parity sample: 512 rows spread over the batch (and over every rank's row block)
    sample = np.arange(0, wl.rows, max(1, wl.rows // 512))[:512]
    want = oracle.rms_norm(oracle.qembedding(wl.qtable, wl.qtype, wl.ids[0][sample], "bf16"), wl.alpha, wl.eps, "bf16")
    sample_t = torch.from_numpy(sample).to(dev)
    mine = (sample >= rb) & (sample < re)
    mine_t = torch.from_numpy(sample[mine] - rb).to(dev)

    def all_ok(flag):
        t = torch.tensor([1.0 if flag else 0.0], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MIN)
        return bool(t.item() == 1.0)

    variants = {}
    # ---- candle's scheme: masked lookup, NCCL sum, norm of every row on every rank ----
    y = emb.forward_rms_norm(ids[0], alpha, wl.eps)
    torch.cuda.synchronize()
    ok_ar = all_ok(np.array_equal(to_oracle(y[sample_t]), want))
    del y
    sampler = ClockSampler(dev.index)
    if rank == 0 and headline:
        sampler.start()
    k = max(2, steps // 2)
    ms_ar = timed(lambda i: emb.forward_rms_norm(ids[i % 2], alpha, wl.eps, check=False), k, 2) / k
    ms_lookup = timed(lambda i: emb.partial(ids[i % 2], check=False, status=st), 4, 2) / 4
    buf = emb.partial(ids[0], check=False, status=st).reshape(-1, wl.hidden)
    dist.all_reduce(as_words(buf))  # the assembled rows: what the norm is timed on
    ms_norm = timed(lambda i: ops.rms_norm(buf, alpha, wl.eps), 4, 2) / 4
    ms_allreduce = timed(lambda i: dist.all_reduce(as_words(buf)), 4, 2) / 4  # (sums of sums: timing only)
    del buf
    variants["all_reduce"] = {
        "ms_per_step": ms_ar, "tokens_per_s": wl.rows / (ms_ar * 1e-3),
        "phases_ms": {"masked_lookup": ms_lookup, "all_reduce": ms_allreduce, "rms_norm": ms_norm},
        "all_reduce_busbw_gbs": 2 * (world - 1) / world * out_bytes / (ms_allreduce * 1e-3) / 1e9,
        "nvlink_out_gbs_per_gpu": 2 * (world - 1) / world * out_bytes / (ms_allreduce * 1e-3) / 1e9,
        "parity": "bit-exact vs unsharded CPU oracle on 512 rows" if ok_ar else "MISMATCH",
        "limiter": "the NCCL all-reduce of the whole [rows, hidden] output (2(N-1)/N of it crosses NVLink per GPU)",
        "note": "candle's scheme: masked lookup (zero bits for foreign rows), NCCL sum over the bit patterns as "
                "32-bit integers, norm of every row on every rank"}
    # ---- the sum as a reduce-scatter, each rank normalises its 1/N of the rows ----
    ys = emb.forward_rms_norm(ids[0], alpha, wl.eps, scatter=True)
    torch.cuda.synchronize()
    ok_rs = all_ok(np.array_equal(to_oracle(ys[mine_t]), want[mine]))
    del ys
    ms_rs = timed(lambda i: emb.forward_rms_norm(ids[i % 2], alpha, wl.eps, scatter=True, check=False), k, 2) / k
    variants["reduce_scatter"] = {
        "ms_per_step": ms_rs, "tokens_per_s": wl.rows / (ms_rs * 1e-3),
        "parity": "bit-exact vs unsharded CPU oracle on this rank's rows of the 512" if ok_rs else "MISMATCH",
        "limiter": "the NCCL reduce-scatter ((N-1)/N of the output per GPU) plus the full-size masked lookup write",
        "note": "each rank ends with its block of the token rows only"}
    torch.cuda.empty_cache()
    # ---- exchange fused into the lookup kernel: peer stores of finished rows ----
    owner_err = None
    try:
        full = [peer_mapped_empty((wl.rows, wl.hidden), torch.bfloat16, dev) for _ in range(2)]
        blocks = [peer_mapped_empty((-(-wl.rows // world), wl.hidden), torch.bfloat16, dev, rank_order=True)
                  for _ in range(2)]
    except Exception as exc:  # symmetric memory unavailable on this system
        owner_err = f"{type(exc).__name__}: {exc}"[:200]
    ok_all = ok_row = True
    e2e = None
    if owner_err is None:
        flag = torch.zeros(1, device=dev)

        # two buffers alternate, so the stores of step i+1 never land in rows a peer still reads from step i
        def owner_all(i):
            emb.forward_rms_norm_owner(ids[i % 2], alpha, wl.eps, full[i % 2][1], status=st)
            dist.all_reduce(flag)  # the ranks' barrier, in stream order: all rows have landed after it

        def owner_row(i):
            emb.forward_rms_norm_row_owner(ids[i % 2], alpha, wl.eps, blocks[i % 2][1], status=st)
            dist.all_reduce(flag)

        owner_all(0)
        torch.cuda.synchronize()
        ok_all = all_ok(np.array_equal(to_oracle(full[0][0][sample_t]), want) and int(st[0].item()) == 0)
        ms_all = timed(owner_all, k, 2) / k
        owner_row(0)
        torch.cuda.synchronize()
        ok_row = all_ok(np.array_equal(to_oracle(blocks[0][0][mine_t]), want[mine]) and int(st[0].item()) == 0)
        ms_row = timed(owner_row, steps, 3) / steps
        sent_all = (world - 1) / world * out_bytes            # owned rows (1/N of all) to N-1 peers
        sent_row = (world - 1) / world / world * out_bytes    # owned rows whose block is another rank's
        # row-owner target: a GPU reads its owned rows' blocks, writes the rows of its own block (local or
        # arriving from peers); NVLink carries sent_row out (and as much in)
        hbm_row = wl.rows * wl.row_qbytes / world + out_bytes / world
        t_row = max(hbm_row / (peak * 1e9), sent_row / 770e9)
        variants["owner_writes_all"] = {
            "ms_per_step": ms_all, "tokens_per_s": wl.rows / (ms_all * 1e-3),
            "nvlink_out_gbs_per_gpu": sent_all / (ms_all * 1e-3) / 1e9,
            "parity": "bit-exact vs unsharded CPU oracle on 512 rows" if ok_all else "MISMATCH",
            "limiter": "peer-store bandwidth: (N-1)/N of the output leaves every GPU and as much arrives",
            "note": "each rank decodes + normalises the rows it owns and stores them into every rank's buffer"}
        variants["row_owner"] = {
            "ms_per_step": ms_row, "tokens_per_s": wl.rows / (ms_row * 1e-3),
            "nvlink_out_gbs_per_gpu": sent_row / (ms_row * 1e-3) / 1e9,
            "target_ms": t_row * 1e3, "frac_of_target": t_row / (ms_row * 1e-3),
            "parity": "bit-exact vs unsharded CPU oracle on this rank's rows of the 512" if ok_row else "MISMATCH",
            "limiter": ("the lookup + norm kernel itself (issue-bound decode of 1/N of the rows); NVLink carries only "
                        "(N-1)/N^2 of the output per GPU"),
            "note": "each finished row is stored only into the buffer of the rank whose row block contains it"}
        # exchange in quantised form: raw block rows routed to the row owner, decoded and normalised there
        routed = RoutedQEmbedding(emb, wl.rows)
        yr = routed.forward_rms_norm(ids[0], alpha, wl.eps, status=st)
        torch.cuda.synchronize()
        ok_routed = all_ok(np.array_equal(to_oracle(yr[mine_t]), want[mine]) and int(st[0].item()) == 0)
        del yr
        ms_routed = timed(lambda i: routed.forward_rms_norm(ids[i % 2], alpha, wl.eps, status=st), steps, 3) / steps
        ms_route_only = timed(lambda i: ops.qembedding_route_rows(
            emb.table, ids[i % 2], routed.staging[i % 2][1],
            [row_shard(wl.rows, r, world)[0] for r in range(world)] + [wl.rows],
            vocab_range=(emb.begin, emb.end), vocab=wl.vocab, status=st), 4, 2) / 4
        sent_q = (world - 1) / world / world * wl.rows * wl.row_qbytes
        hbm_routed = (2 * wl.rows * wl.row_qbytes + wl.rows * wl.row_qbytes + out_bytes) / world
        t_routed = max(hbm_routed / (peak * 1e9), sent_q / 770e9)
        variants["routed_rows"] = {
            "ms_per_step": ms_routed, "tokens_per_s": wl.rows / (ms_routed * 1e-3),
            "phases_ms": {"route_raw_rows": ms_route_only, "barrier_then_local_lookup_norm": ms_routed - ms_route_only},
            "nvlink_out_gbs_per_gpu": sent_q / (ms_route_only * 1e-3) / 1e9,
            "target_ms": t_routed * 1e3, "frac_of_target": t_routed / (ms_routed * 1e-3),
            "parity": "bit-exact vs unsharded CPU oracle on this rank's rows of the 512" if ok_routed else "MISMATCH",
            "limiter": ("the local lookup + norm kernel (issue-bound decode of 1/N of the rows) plus one barrier; NVLink "
                        "carries only (N-1)/N^2 of the QUANTISED rows per GPU"),
            "note": "raw block rows are routed to the rank whose row block holds them and decoded there"}
        ok_row = ok_row and ok_routed
        # end to end for the routed variant: ids from pinned host memory, this rank's block back to the host
        host_ids = [torch.from_numpy(np.ascontiguousarray(i.reshape(-1)).view(np.int32)).pin_memory() for i in wl.ids]
        dev_ids = torch.empty_like(ids[0].reshape(-1))
        host_out = torch.empty(re - rb, wl.hidden, dtype=torch.bfloat16).pin_memory()

        def e2e_step(i):
            dev_ids.view(torch.uint8).copy_(host_ids[i % 2].view(torch.uint8), non_blocking=True)
            host_out.copy_(routed.forward_rms_norm(dev_ids, alpha, wl.eps, status=st), non_blocking=True)

        ke = max(2, min(steps, 5))
        ms_e2e = timed(e2e_step, ke, 1) / ke
        e2e = {"value": wl.rows / (ms_e2e * 1e-3), "unit": "tokens/s", "ms_per_step": ms_e2e,
               "h2d_bytes_per_step": int(dev_ids.numel() * dev_ids.element_size()) * world,
               "d2h_bytes_per_step": out_bytes,
               "how": "routed-rows variant: every rank uploads the ids; each rank downloads its block of the finished rows"}
    else:
        variants["owner_writes_all"] = variants["row_owner"] = variants["routed_rows"] = {"unavailable": owner_err}
    clocks = sampler.stop() if (rank == 0 and headline) else None
    parity_ok = ok_ar and ok_rs and ok_all and ok_row
    best = min((v for v in variants.values() if "ms_per_step" in v), key=lambda v: v["ms_per_step"])
    best_name = [n for n, v in variants.items() if v is best][0]
    entry = {"workload": wl.desc, "rows": wl.rows, "n_gpus": world, "scaling": "strong", "variants": variants,
             "fastest_variant": best_name, "ms_per_step": best["ms_per_step"], "tokens_per_s": best["tokens_per_s"],
             "e2e": e2e, "parity": "bit-exact vs unsharded CPU oracle" if parity_ok else "MISMATCH"}
    if not headline:
        return entry, parity_ok
    hbm_best = {"routed_rows": (3 * wl.rows * wl.row_qbytes + out_bytes) / world}.get(
        best_name, wl.rows * wl.row_qbytes / world + out_bytes / world)
    roof = ({"bound": "hbm", "achieved": hbm_best / (best["ms_per_step"] * 1e-3) / 1e9,
             "peak": peak, "unit": "GB/s", "frac": best["frac_of_target"], "peak_kind": "of measured", "traffic": None,
             "note": f"{best_name} variant: target time = max(per-GPU HBM bytes / measured HBM peak, bytes leaving the "
                     "GPU / 770 GB/s measured peer-copy bandwidth); frac = target / achieved time"}
            if "frac_of_target" in best else None)
    line = {"metric": METRIC, "value": best["tokens_per_s"], "unit": "tokens/s", "n_gpus": world, "steps": steps,
            "warmup": args.warmup, "ms_per_step": best["ms_per_step"], "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic (seed 0)",
            "config": config_of(wl, world, f"vocab sharded x{world}; fastest variant: {best_name}"),
            "roofline": roof, "e2e": e2e, "gpu_launches": steps, "clocks": clocks}
    line.update({k2: v for k2, v in entry.items() if k2 in ("variants", "fastest_variant", "parity")})
    return line, parity_ok


# ------------------------------------------------------------------------------------------------
# CPU arm: the oracle, threaded the way candle threads its CPU backend
# ------------------------------------------------------------------------------------------------
def cpu_flow(wl, rows, threads):
    """One pass of candle's CPU flow over `rows` token rows; returns seconds (and one-off load seconds)."""
    import oracle

    load_s = 0.0
    if wl.name == "c1":
        ids = wl.ids[0][:rows]
        t0 = time.perf_counter()
        e = oracle.index_select(wl.table, ids, 0)  # single-threaded in candle
        y = oracle.rms_norm(e, wl.alpha, wl.eps, "f32", threads=threads)  # rayon: one task per row
        dt = time.perf_counter() - t0
    elif wl.name in ("c3", "c4"):
        # candle dequantises the whole table once at load (single-threaded) and casts it to bf16;
        # time that on a 1/16 slice of the vocabulary and scale, then gather + norm per batch
        slice_rows = wl.vocab // 16
        t0 = time.perf_counter()
        f32 = oracle.dequantize(wl.qtable[:slice_rows], wl.qtype, threads=1)
        tbl = oracle.cast_from_f32(f32, "bf16", threads=1)
        load_s = (time.perf_counter() - t0) * 16
        ids = (wl.ids[0][:rows] % slice_rows).astype(np.uint32)
        t0 = time.perf_counter()
        e = oracle.index_select(tbl, ids, 0)
        y = oracle.rms_norm(e, wl.alpha, wl.eps, "bf16", threads=threads)
        dt = time.perf_counter() - t0
    else:
        reps = -(-rows // wl.x[0].shape[0])
        x = np.tile(wl.x[0], (reps, 1))[:rows]
        r = np.tile(wl.res[0], (reps, 1))[:rows]
        t0 = time.perf_counter()
        h = oracle.add(x, r, "bf16", threads=1)  # candle's binary map is sequential
        if wl.name == "c2":
            y = oracle.layer_norm(h, wl.gamma, wl.beta, wl.eps, "bf16", threads=threads)
        else:
            y = oracle.rms_norm(h, wl.alpha, wl.eps, "bf16", threads=threads)
        dt = time.perf_counter() - t0
    del y
    return dt, load_s


LOAD_NOTE = "timed on 1/16 of the vocabulary (dequantise + cast, one thread) and multiplied by 16"


def cpu_baseline(wl, budget_s=15.0):
    cores = host_cores()
    rows = min(wl.rows, 2048)
    dt, load_s = cpu_flow(wl, rows, cores)  # warm-up + calibration
    rows = int(min(wl.rows, max(rows, rows * (budget_s / 3) / max(dt, 1e-4))))
    times = []
    for _ in range(3):
        dt, _ = cpu_flow(wl, rows, cores)
        times.append(dt)
    dt = statistics.median(times)
    out = {"value": rows / dt, "unit": "tokens/s", "cores": cores, "kind": "port",
           "sample": f"{rows} of {wl.rows} token rows of the same workload, median of 3; norms on {cores} threads, "
                     f"gather/add/dequant/cast on 1 thread as candle does"}
    if load_s:
        out["one_off_table_load_s"] = load_s
        out["one_off_table_load_how"] = LOAD_NOTE
    return out


def reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    world = args.gpus
    wl = Workload(args.workload, args.rows_scale)
    cores = host_cores()
    rows = min(wl.rows, 4096)
    dt, load_s = cpu_flow(wl, rows, cores)
    # size a step so that warmup + steps stay within a few minutes
    per_step_budget = min(20.0, 150.0 / max(1, args.steps + args.warmup))
    rows = int(min(wl.rows, max(256, rows * per_step_budget / max(dt, 1e-4))))
    for _ in range(args.warmup):
        cpu_flow(wl, rows, cores)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        cpu_flow(wl, rows, cores)
    total = time.perf_counter() - t0
    value = rows * args.steps / total
    sample = (f"each step = {rows} of {wl.rows} token rows; norms on {cores} threads, gather/add/dequant/cast "
              f"single-threaded as in candle's CPU backend")
    base = {"value": value, "unit": "tokens/s", "cores": cores, "kind": "port", "sample": sample,
            "note": "candle is Rust and cannot be built in this image; this is the C restatement of its CPU code "
                    "(oracle/)"}
    if load_s:
        base["one_off_table_load_s"] = load_s
        base["one_off_table_load_how"] = LOAD_NOTE
    parallelism = f"vocab sharded x{world}" if wl.name == "c4" else None
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": value,
        "unit": "tokens/s", "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": total / args.steps * 1e3, "higher_is_better": True,
        "scaling": "strong" if wl.name == "c4" else "weak", "vs_baseline": None,
        "dtype": wl.dtype, "data": "synthetic (seed 0)",
        "config": config_of(wl, world, parallelism),
        "cpu_baseline": base,
        "e2e": {"value": value, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--workload", default="c5", choices=["c1", "c2", "c3", "c4", "c5", "next"],
                    help="'next' runs only the operators next to the hot path (one GPU) and prints their record")
    ap.add_argument("--no-sweep", action="store_true", help="skip the brief runs of the other workloads")
    ap.add_argument("--rows-scale", type=float, default=1.0, help="c4 / c5 only: fraction of the configured rows")
    ap.add_argument("--impl", default="candle_b200", choices=["candle_b200", "reference"])
    ap.add_argument("--no-cpu", action="store_true", help="skip the cpu_baseline leg")
    args = ap.parse_args()
    if args.warmup < 3 and args.impl != "reference":
        args.warmup = 3
    if args.impl == "reference":
        reference_arm(args)
    else:
        gpu_arm(args)


if __name__ == "__main__":
    main()
