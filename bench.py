"""Benchmark of the embed + norm hot path on B200, next to candle's CPU path on the host cores.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload c1|c2|c3|c4|c5] [--impl reference]

One "step" is one pass of the hot path over one batch of synthetic token rows.  The default
workload is the largest single-GPU configuration and the one the row-sharded scaling target is
stated on: C5, RMSNorm + fused residual add, bf16, hidden 8192, 65536 token rows (3.2 GB of
compulsory HBM traffic per step).  Token rows are independent, so N GPUs each run the same number
of rows (weak scaling, no collective); C4 is the vocab-sharded exception and needs N >= 2.  At
N = 1 the other single-GPU configurations (C1, C2, C3) are measured briefly in the same run and
reported under "other_workloads".

Rank 0 prints ONE JSON line.  `value` is token rows per second with the inputs resident in HBM;
`e2e` is the same through the public front end with ids coming from pinned host memory and the
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

# dram__bytes_read.sum + dram__bytes_write.sum per launch from the ncu captures summarised under
# profiles/ (null until a capture of that kernel exists)
# c5: 364.5 MB measured on the 8192-row capture, scaled x8 (traffic grows with rows);
# see profiles/rms_rowreg_kernel__c5_rmsnorm_residual_bf16_h8192.md
NCU_TRAFFIC_BYTES = {"c3": None, "c5": 2916000000, "c2": None, "c1": None, "c4": None}


def measured_peak():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


# ------------------------------------------------------------------------------------------------
# workloads: seeded synthetic inputs with the shapes and value distributions of the configs
# ------------------------------------------------------------------------------------------------
def zipf_ids(rng, vocab, n, s=1.1):
    p = 1.0 / np.arange(1, vocab + 1, dtype=np.float64) ** s
    p /= p.sum()
    return rng.choice(vocab, size=n, p=p).astype(np.uint32)  # rank k -> id k-1


class Workload:
    """Holds host-side inputs (numpy, oracle layout) and knows its algorithmic bytes per step."""

    def __init__(self, name, rows_scale=1.0):
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
                self.desc = ("C3 GGUF Q8_0 embedding 128256x4096 -> bf16 -> RMSNorm eps 1e-5, ids Zipf(1.1) 32x2048 "
                             "(rank k -> id k-1)")
                self.vocab, self.hidden, self.rows, self.qtype = 128256, 4096, 32 * 2048, "q8_0"
            else:
                self.desc = ("C4 GGUF Q4_0 embedding 152064x8192 vocab-sharded, ids uniform 64x4096, masked lookup + "
                             "all-reduce + RMSNorm eps 1e-5")
                self.vocab, self.hidden, self.rows, self.qtype = 152064, 8192, 64 * 4096, "q4_0"
            self.dtype = "bf16"
            self.qtable = make_qtable(rng, self.qtype, self.vocab, self.hidden)
            self.alpha = randn(rng, (self.hidden,), "bf16", 1.0, 0.1)
            self.n_sets = 2
            gen = (lambda: zipf_ids(rng, self.vocab, self.rows)) if name == "c3" else (
                lambda: rng.integers(0, self.vocab, size=self.rows).astype(np.uint32))
            self.ids = [gen() for _ in range(self.n_sets)]
            self.row_qbytes = self.qtable.shape[1]
            self.bytes_per_step = self.rows * (self.row_qbytes + self.hidden * 2)
            self.eps = 1e-5
        elif name == "c5":
            self.rows = int(65536 * rows_scale)
            self.desc = f"C5 RMSNorm + residual bf16, hidden 8192, {self.rows} token rows, eps 1e-5"
            self.hidden, self.dtype = 8192, "bf16"
            self.n_sets = 1 if 3 * self.rows * 8192 * 2 > 4 * L2_BYTES else 8
            base = min(self.rows, 4096)  # seeded block, tiled to the full row count
            self.x = [randn(rng, (base, self.hidden), "bf16") for _ in range(1)]
            self.res = [randn(rng, (base, self.hidden), "bf16") for _ in range(1)]
            self.alpha = randn(rng, (self.hidden,), "bf16", 1.0, 0.1)
            self.bytes_per_step = 3 * self.rows * self.hidden * 2
            self.eps = 1e-5
        else:
            raise SystemExit(f"unknown workload {name}")


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
    """Device-resident inputs of one workload plus the closures that launch it."""

    def __init__(self, wl, dev, stream, st):
        import torch

        import candle_b200 as cb
        from candle_b200 import _cabi
        from helpers import from_oracle, ids_tensor, to_oracle
        import oracle

        self.wl, S = wl, wl.n_sets
        if wl.name == "c1":
            table = from_oracle(wl.table, wl.dtype, dev)
            alpha = from_oracle(wl.alpha, wl.dtype, dev)
            ids = [ids_tensor(i, dev) for i in wl.ids]
            ys = [torch.empty(wl.rows, wl.hidden, dtype=table.dtype, device=dev) for _ in range(S)]

            def launch(ids_ptr, y):
                _cabi.call("cb200_embedding_rms_norm", table.data_ptr(), ids_ptr, alpha.data_ptr(), y.data_ptr(), None,
                           wl.vocab, wl.hidden, wl.rows, wl.eps, 0, 1, 0, st.data_ptr(), stream.cuda_stream)

            self.step = lambda i: launch(ids[i % S].data_ptr(), ys[i % S])
            self.check = lambda: np.array_equal(
                to_oracle(ys[0][:512]),
                oracle.rms_norm(oracle.embedding(wl.table, wl.ids[0][:512]), wl.alpha, wl.eps, "f32"))
            host_in = [torch.from_numpy(i.view(np.int32)).pin_memory() for i in wl.ids]
            dev_in = torch.empty(wl.rows, dtype=torch.int32, device=dev)

            def e2e_step(i, host_out):
                dev_in.copy_(host_in[i % S], non_blocking=True)
                launch(dev_in.data_ptr(), ys[0])
                host_out.copy_(ys[0], non_blocking=True)
            self.h2d = wl.rows * 4
        elif wl.name == "c3":
            q = cb.QTensor.from_raw(torch.from_numpy(wl.qtable), cb.GgmlDType.Q8_0, (wl.vocab, wl.hidden), device=dev)
            alpha = from_oracle(wl.alpha, "bf16", dev)
            ids = [ids_tensor(i, dev) for i in wl.ids]
            ys = [torch.empty(wl.rows, wl.hidden, dtype=torch.bfloat16, device=dev) for _ in range(S)]

            def launch(ids_ptr, y):
                _cabi.call("cb200_qembedding_rms_norm", q.data.data_ptr(), q.dtype.value, ids_ptr, alpha.data_ptr(),
                           y.data_ptr(), None, wl.vocab, wl.hidden, wl.rows, wl.eps, 2, 1, 0, wl.vocab, 0,
                           st.data_ptr(), stream.cuda_stream)

            self.step = lambda i: launch(ids[i % S].data_ptr(), ys[i % S])
            self.check = lambda: np.array_equal(
                to_oracle(ys[0][:512]),
                oracle.rms_norm(oracle.qembedding(wl.qtable, wl.qtype, wl.ids[0][:512], "bf16"), wl.alpha, wl.eps, "bf16"))
            host_in = [torch.from_numpy(i.view(np.int32)).pin_memory() for i in wl.ids]
            dev_in = torch.empty(wl.rows, dtype=torch.int32, device=dev)

            def e2e_step(i, host_out):
                dev_in.copy_(host_in[i % S], non_blocking=True)
                launch(dev_in.data_ptr(), ys[0])
                host_out.copy_(ys[0], non_blocking=True)
            self.h2d = wl.rows * 4
        else:  # c2 / c5: dense rows + residual
            reps = -(-wl.rows // wl.x[0].shape[0])
            xs, rs, ys = [], [], []
            for s in range(S):
                bx = from_oracle(wl.x[s % len(wl.x)], "bf16", dev)
                br = from_oracle(wl.res[s % len(wl.res)], "bf16", dev)
                xs.append(bx.repeat(reps, 1)[: wl.rows].contiguous())
                rs.append(br.repeat(reps, 1)[: wl.rows].contiguous())
                ys.append(torch.empty(wl.rows, wl.hidden, dtype=torch.bfloat16, device=dev))
            n = min(512, wl.x[0].shape[0])
            h = oracle.add(wl.x[0][:n], wl.res[0][:n], "bf16")
            if wl.name == "c2":
                g, b = from_oracle(wl.gamma, "bf16", dev), from_oracle(wl.beta, "bf16", dev)

                def launch(x, r, y):
                    _cabi.call("cb200_layer_norm", x.data_ptr(), r.data_ptr(), g.data_ptr(), b.data_ptr(), y.data_ptr(),
                               None, wl.rows, wl.hidden, wl.eps, 2, 0, stream.cuda_stream)
                self.check = lambda: np.array_equal(
                    to_oracle(ys[0][:n]), oracle.layer_norm(h, wl.gamma, wl.beta, wl.eps, "bf16"))
            else:
                a = from_oracle(wl.alpha, "bf16", dev)

                def launch(x, r, y):
                    _cabi.call("cb200_rms_norm", x.data_ptr(), r.data_ptr(), a.data_ptr(), y.data_ptr(), None, wl.rows,
                               wl.hidden, wl.eps, 2, 0, stream.cuda_stream)
                self.check = lambda: np.array_equal(to_oracle(ys[0][:n]), oracle.rms_norm(h, wl.alpha, wl.eps, "bf16"))
            self.step = lambda i: launch(xs[i % S], rs[i % S], ys[i % S])
            host_x, host_r = xs[0].cpu().pin_memory(), rs[0].cpu().pin_memory()

            # end to end through the library's pinned-host front end: rows in chunks, copy in / kernel /
            # copy out overlapped on three streams
            pipe = cb.PinnedNormPipeline(wl.hidden, torch.bfloat16, dev, chunk_rows=max(1024, wl.rows // 8))
            self.e2e_note = f"PinnedNormPipeline, chunks of {pipe.chunk_rows} rows on three streams"

            def e2e_step(i, host_out):
                if wl.name == "c2":
                    pipe.run(host_x, host_out, g, wl.eps, residual_host=host_r, beta=b)
                else:
                    pipe.run(host_x, host_out, a, wl.eps, residual_host=host_r)
            self.h2d = 2 * wl.rows * wl.hidden * 2
        self.e2e_step = e2e_step
        self.out_dtype = ys[0].dtype


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
        dist.init_process_group("nccl", device_id=dev)
    if args.workload == "c4":
        from candle_b200 import parallel

        return parallel.bench_c4(args, rank, world, dev)

    stream = torch.cuda.current_stream()
    st = new_status(dev)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, steps, warmup):
        for i in range(warmup):
            fn(i)
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for i in range(steps):
            fn(warmup + i)
        e1.record(stream)
        barrier()
        ms = e0.elapsed_time(e1)
        if world > 1:
            t = torch.tensor([ms], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = t.item()
        return ms

    wl = Workload(args.workload, args.rows_scale)
    run = Runner(wl, dev, stream, st)

    # ---- parity spot check on this very workload before anything is timed ----
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
    barrier()
    raise_for_status(st)

    # ---- end to end: host buffers in, host rows out, through the same call ----
    host_out = torch.empty(wl.rows, wl.hidden, dtype=run.out_dtype).pin_memory()
    e2e_steps = max(2, min(args.steps, 10))
    e2e_ms = timed(lambda i: run.e2e_step(i, host_out), e2e_steps, 1)
    d2h = host_out.numel() * host_out.element_size()
    e2e_how = getattr(run, "e2e_note", "one call per step: ids from pinned host memory in, rows to pinned host memory out")

    peak, peak_kind = measured_peak()
    others = {}
    if world == 1 and not args.no_sweep:
        del run, host_out
        torch.cuda.empty_cache()
        for name in ("c1", "c2", "c3", "c5"):
            if name == wl.name:
                continue
            w2 = Workload(name)
            r2 = Runner(w2, dev, stream, st)
            r2.step(0)
            torch.cuda.synchronize()
            ok2 = bool(r2.check())
            k = 20
            ms2 = timed(r2.step, k, 3) / k
            gbs = w2.bytes_per_step / (ms2 * 1e-3) / 1e9
            others[name] = {"workload": w2.desc, "ms_per_step": ms2, "tokens_per_s": w2.rows / (ms2 * 1e-3),
                            "achieved_gbs": gbs, "frac_of_measured_peak": gbs / peak,
                            "parity": "bit-exact on 512 rows" if ok2 else "MISMATCH"}
            parity_ok = parity_ok and ok2
            del r2, w2
            torch.cuda.empty_cache()

    if rank == 0:
        ms_per_step = ms / args.steps
        achieved = wl.bytes_per_step / (ms_per_step * 1e-3) / 1e9
        out = {
            "metric": "tokens/s, embed+norm (HBM GB/s in roofline)",
            "value": world * wl.rows * args.steps / (ms * 1e-3),
            "unit": "tokens/s",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_per_step,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": wl.dtype, "data": "synthetic (seed 0)",
            "config": {"workload": wl.desc, "rows_per_gpu": wl.rows, "hidden": wl.hidden,
                       "parallelism": f"token rows x{world}, no collective",
                       "l2": f"rotating {wl.n_sets} buffer set(s); working set per step "
                             f"{wl.bytes_per_step / 1e6:.0f} MB vs 126 MB L2"},
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                         "peak_kind": f"of {peak_kind}", "frac_of_nominal_8000": achieved / 8000.0,
                         "algorithmic_bytes_per_launch": wl.bytes_per_step,
                         "traffic": NCU_TRAFFIC_BYTES.get(wl.name)},
            "e2e": {"value": world * wl.rows * e2e_steps / (e2e_ms * 1e-3), "unit": "tokens/s",
                    "h2d_bytes_per_step": run_h2d(wl), "d2h_bytes_per_step": d2h, "ms_per_step": e2e_ms / e2e_steps,
                    "how": e2e_how},
            "gpu_launches": args.steps,
            "parity": "bit-exact vs CPU oracle on the first 512 rows" if parity_ok else "MISMATCH vs CPU oracle",
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


def cpu_baseline(wl, budget_s=15.0):
    import oracle

    cores = oracle.max_threads()
    rows = min(wl.rows, 2048)
    dt, load_s = cpu_flow(wl, rows, cores)  # warm-up + calibration
    rows = int(min(wl.rows, max(rows, rows * (budget_s / 3) / max(dt, 1e-4))))
    times = []
    for _ in range(3):
        dt, _ = cpu_flow(wl, rows, cores)
        times.append(dt)
    dt = statistics.median(times)
    return {"value": rows / dt, "unit": "tokens/s", "cores": cores, "kind": "port",
            "sample": f"{rows} of {wl.rows} token rows of the same workload, median of 3; norms on {cores} threads, "
                      f"gather/add/dequant/cast on 1 thread as candle does",
            "one_off_table_load_s": load_s or None}


def reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    import oracle

    wl = Workload(args.workload if args.workload != "c4" else "c4", args.rows_scale)
    cores = oracle.max_threads()
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
    print(json.dumps({
        "impl": "reference", "metric": "tokens/s, embed+norm (HBM GB/s in roofline)", "value": value,
        "unit": "tokens/s", "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": total / args.steps * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": wl.dtype, "data": "synthetic (seed 0)",
        "config": {"workload": wl.desc, "rows_per_step": rows, "hidden": wl.hidden},
        "cpu_baseline": {"value": value, "unit": "tokens/s", "cores": cores, "kind": "port", "sample": sample,
                         "one_off_table_load_s": load_s or None,
                         "note": "candle is Rust and cannot be built in this image; this is the C restatement of "
                                 "its CPU code (oracle/)"},
        "e2e": {"value": value, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--workload", default="c5", choices=["c1", "c2", "c3", "c4", "c5"])
    ap.add_argument("--no-sweep", action="store_true", help="skip the brief runs of the other workloads")
    ap.add_argument("--rows-scale", type=float, default=1.0, help="c5 only: fraction of 65536 rows")
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
