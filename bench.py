#!/usr/bin/env python
"""Decode throughput of the PowerInfer hot path on B200: one JSON line per run.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--config NAME] [--batch T]

A step is one decode token for each of T sequences (T = 1 for the headline) of the ReLU-Llama-2-70B-shaped Q4_0
model (80 layers, d 8192, FFN 28672, 64/8 heads, rank-1024 FP16 predictors firing 12 % on a Zipf profile), after a
256-token prompt.  Weights are seeded random draws made on the device (there are no checkpoints), sharded by FFN
neuron and attention head when N > 1.

value     tokens/s with the step's inputs resident in HBM: K x (CUDA-graph step + on-device greedy feedback),
          CUDA events on the engine's stream, barrier + synchronize on both sides, max over ranks.
e2e       the same through the host-buffer C-ABI call (pi_engine_decode_host = llama_decode + llama_get_logits):
          token ids and positions copied host->device, the full logits and the greedy id copied back, every step.
roofline  the kernel class that takes the largest share of the step: that stage's kernels for all layers are replayed back
          to back from a CUDA graph (launched exactly as inside a step) between two CUDA events; achieved = algorithmic
          bytes (active rows only) / mean launch time.  `stage_ms_profiled` is a second view: events around every single
          launch of a step, which serialises the kernels (no overlap) and therefore sums to more than the step.
cpu_baseline / --impl reference
          the reference's own CPU code (oracle/_ref: its ggml.c compiled unmodified) running the per-layer mat-vecs
          and sparse operators of the same shape on all host cores, extrapolated over the layers.
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


def measured_peaks():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            p = json.load(f)
        return float(p["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


def ncu_traffic(cfg_name: str) -> dict:
    """DRAM bytes per launch (dram__bytes_read.sum + dram__bytes_write.sum) of each stage's kernels, from the ncu capture
    of the 4-layer case of the same layer shape (traffic per launch does not depend on the layer count).  The figures
    live in a text file next to the ncu summaries, one `stage bytes` pair per line after a header naming the commit they
    were captured at; a stage whose kernel changed since is simply absent there and reports null."""
    out = {}
    try:
        with open(os.path.join(ROOT, "profiles", f"dram_traffic_{cfg_name}.txt")) as f:
            for line in f:
                parts = line.split()
                if len(parts) >= 2 and not line.startswith("#"):
                    out[parts[0]] = float(parts[1])
    except OSError:
        pass
    return out


def physical_cores() -> int:
    try:
        import psutil
        n = psutil.cpu_count(logical=False)
        if n:
            return int(n)
    except Exception:
        pass
    return os.cpu_count() or 1


def pi_env() -> dict:
    """Every PI_* switch in effect: a line with an empty dict ran the default kernels."""
    return {k: v for k, v in sorted(os.environ.items()) if k.startswith("PI_")}

# ------------------------------------------------------------------------------------------------ clocks

class ClockSampler:
    """nvidia-smi clocks and throttle reasons sampled every 50 ms; `stop(t0, t1)` keeps the samples that arrived while the
    timed region ran (host clock around it: from the first launch to the end of the synchronisation that follows it)."""
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.rows, self.proc = [], None
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                                          "-lms", "50", "-i", str(index)], stdout=subprocess.PIPE, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append((time.monotonic(), [c.strip() for c in line.split(",")]))

    def stop(self, t0: float | None = None, t1: float | None = None) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.1)                                    # let the last line of the region arrive
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            pass
        sm, mx, reasons = [], [], set()
        inside = [r for (t, r) in self.rows if t0 is not None and t1 is not None and t0 <= t <= t1 + 0.05]
        for r in (inside if inside else [r for (_, r) in self.rows]):
            try:
                sm.append(float(r[0])); mx.append(float(r[1]))
            except Exception:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


# ------------------------------------------------------------------------------------------------ CPU reference arm

def cpu_reference(spec, n_threads: int | None = None) -> dict:
    """Times the reference's CPU operators (its own ggml.c, through oracle/_ref/libpi_ref.so) on ONE layer of the
    configuration plus the lm head, all host threads, and extrapolates over the layers."""
    import numpy as np
    from oracle import pio
    from powerinfer_b200 import synth
    ref = pio.Ref()
    nth = n_threads or physical_cores()
    rng = np.random.default_rng(0)
    d, F, R, dkv = spec.d, spec.n_ff, spec.rank, spec.d_kv
    q4 = spec.wtype == synth.Q4_0

    def weight(rows):
        w = rng.standard_normal((rows, d), dtype=np.float32) * np.float32(spec.sigma)
        return ref.quantize_q4_0(w) if q4 else w.astype(np.float16)

    rb = (d // 32 * 18) if q4 else d                 # row length in array elements (bytes for Q4_0, halves for F16)
    big = np.asarray(weight(F)).reshape(F, rb)       # one draw, tiled: values do not affect the timing
    rows_of = lambda rows: np.ascontiguousarray(np.resize(big, (rows, rb)))
    up, gate, down = big, big.copy(), big.copy()
    wqkv, wo = rows_of(d + 2 * dkv), rows_of(d)
    n_lm = spec.n_vocab
    lm = rows_of(n_lm)
    fc1 = (rng.standard_normal((R, d), dtype=np.float32) * 0.02).astype(np.float16)
    fc2 = (rng.standard_normal((F, R), dtype=np.float32) * 0.02).astype(np.float16)
    x = rng.standard_normal((1, d), dtype=np.float32)
    hid = np.abs(rng.standard_normal((1, R), dtype=np.float32))
    prof = synth.zipf_profile(F, spec.firing)[rng.permutation(F)]
    idx = np.where(rng.random((1, F)) < prof, 1.0, -1.0).astype(np.float32)
    h = np.abs(rng.standard_normal((1, F), dtype=np.float32)) * (idx > 0)
    wt = spec.wtype
    t = {}
    reps = 3
    ref.mul_mat(wt, wqkv, d + 2 * dkv, d, x, nth, reps); t["qkv"] = ref.last_time
    ref.mul_mat(wt, wo, d, d, x, nth, reps); t["out_proj"] = ref.last_time
    ref.mul_mat(synth.F16, fc1, R, d, x, nth, reps); t["predictor"] = ref.last_time
    ref.mul_mat(synth.F16, fc2, F, R, hid, nth, reps); t["predictor"] += ref.last_time
    ref.mul_mat_idx(wt, up, F, d, x, idx, None, spec.threshold, nth, reps); t["up_gate"] = ref.last_time
    if spec.arch == synth.ARCH_LLAMA:
        ref.mul_mat_idx(wt, gate, F, d, x, idx, None, spec.threshold, nth, reps); t["up_gate"] += ref.last_time
    ref.axpy(wt, down, F, d, h, idx, None, spec.threshold, nth, reps); t["down"] = ref.last_time
    ref.mul_mat(wt if spec.arch != synth.ARCH_OPT else synth.F16, lm if spec.arch != synth.ARCH_OPT else np.zeros((n_lm, d), np.float16), n_lm, d, x, nth, reps); t_lm = ref.last_time
    per_layer = sum(t.values())
    per_token = per_layer * spec.n_layer + t_lm
    return {"value": 1.0 / per_token, "unit": "tok/s", "cores": nth, "kind": "reference",
            "sample": f"reference ggml CPU ops (oracle/_ref, AVX2 build) for 1 of {spec.n_layer} layers "
                      f"(qkv, out-proj, predictor, mul_mat_idx up/gate, axpy down) + lm head at the config's shape, best of {reps}, "
                      f"{nth} threads (the machine's physical cores), extrapolated x{spec.n_layer}; attention/norm/RoPE nodes not included",
            "ms_per_layer": {k: round(v * 1e3, 4) for k, v in t.items()}, "ms_per_token": per_token * 1e3}


def cpu_reference_decode(spec, n_threads: int | None = None) -> dict:
    """The reference's OWN decode loop (its unmodified llama.cpp + ggml.c, oracle/_ref/ref_decode: llama_decode ->
    llm_build_ffn_sparse -> ggml_graph_compute, every node on the host cores) on models of the configuration's layer shape
    with 1 and 3 layers; time per token = a + b x layers, read off the two runs and extended to the configuration's layer
    count.  Seeded synthetic weights (Q4_0 blocks drawn directly: the time does not depend on the values)."""
    import dataclasses
    import re
    import tempfile
    import numpy as np
    from powerinfer_b200 import gguf_loader, synth
    exe = os.path.join(ROOT, "oracle", "_ref", "ref_decode")
    if not os.path.exists(exe):
        raise FileNotFoundError(exe)
    nth = n_threads or physical_cores()
    n_prompt, n_steps = 4, 7
    per_token = {}
    with tempfile.TemporaryDirectory() as td:
        for L in (1, 3):
            sp = dataclasses.replace(spec, n_layer=L, n_ctx=64)
            path = os.path.join(td, f"m{L}.gguf")
            gguf_loader.write_model_file(sp, synth.build_model(sp, fast_q4=True), path)
            tp, op = os.path.join(td, "tok.i32"), os.path.join(td, "out.f32")
            np.random.default_rng(0).integers(3, sp.n_vocab, n_prompt + n_steps).astype(np.int32).tofile(tp)
            r = subprocess.run([exe, path, tp, str(n_prompt), str(n_steps), str(nth), op, "single", "forced"], capture_output=True, text=True, check=True)
            m = re.search(r"ref_decode: (\d+) decode steps in ([0-9.]+) ms", r.stderr)
            per_token[L] = float(m.group(2)) / int(m.group(1)) * 1e-3
            os.remove(path)
    b = (per_token[3] - per_token[1]) / 2.0
    a = per_token[1] - b
    t = a + b * spec.n_layer
    return {"value": 1.0 / t, "unit": "tok/s", "cores": nth, "kind": "reference",
            "sample": f"the reference's llama_decode loop (oracle/_ref/ref_decode, AVX2 build, {nth} threads = physical cores) on 1- and 3-layer "
                      f"models of the configuration's layer shape, {n_steps - 1} decode steps each after a {n_prompt}-token prompt; "
                      f"seconds per token {per_token[1]:.4f} and {per_token[3]:.4f} -> {a:.4f} + {b:.4f} x layers, extended to {spec.n_layer} layers",
            "ms_per_token": t * 1e3, "ms_per_layer": b * 1e3, "ms_fixed": a * 1e3}


# ------------------------------------------------------------------------------------------------ sparse-FFN microbench

def sparse_ffn_microbench(args):
    """One sparse-FFN layer at the Llama-2-13B shape (d 5120, F 13824), FP16 and Q4_0 rows, mean sparsity 50/80/90/95 %
    under a Zipf(1.1) per-neuron profile, batch 1/4/8/16 with a union mask: ggml_mul_mat_idx (up), ggml_axpy (down) and the
    whole FFN (up + gate + glue + down) through the C ABI.  Every timed launch sequence rotates over enough distinct copies
    of the weights that the active rows of consecutive iterations exceed twice the L2 capacity, and is replayed from a
    CUDA graph so that the host's call overhead is not what is measured.  Bytes: active rows x row bytes per matrix
    + T*d*4 + T*F*4 (the algorithmic bytes; inactive rows are never read)."""
    import numpy as np
    import torch
    from powerinfer_b200 import ggml_ops as g, synth
    torch.cuda.set_device(0)
    d, F = 5120, 13824
    peak, peak_kind = measured_peaks()
    reps = max(3, min(args.steps, 20))
    rng = np.random.default_rng(0)
    gen = torch.Generator(device="cuda"); gen.manual_seed(0)
    base = [(torch.randn(F, d, device="cuda", generator=gen) * 0.02).to(torch.float16) for _ in range(3)]
    table = []
    only = args.only.split(":") if args.only else None
    for wtype, wname in ((synth.F16, "F16"), (synth.Q4_0, "Q4_0")):
        if only and only[0] != wname:
            continue
        rowb = 2 * d if wtype == synth.F16 else d // 32 * 18
        n_copies = 12 if wtype == synth.F16 else 44          # 95 % sparse: 12 x 21 MB / 44 x 6 MB of active rows > 2 x 126 MB
        if wtype == synth.F16:
            one = [g.Weight(wtype, b.view(torch.uint8).reshape(-1), F, d) for b in base]
        else:
            one = []
            for b in base:
                raw = g.quantize_q4_0(b.float())
                dev = torch.empty_like(raw)
                from powerinfer_b200._lib import check, lib
                check(lib.pi_q4_0_repack(raw.data_ptr(), dev.data_ptr(), F, d, torch.cuda.current_stream().cuda_stream))
                one.append(g.Weight(wtype, dev, F, d))
        copies = [[g.Weight(wtype, w.data.clone(), F, d) for w in one] for _ in range(n_copies)]
        for sparsity in (0.5, 0.8, 0.9, 0.95):
            prof = synth.zipf_profile(F, 1.0 - sparsity)[rng.permutation(F)]
            for T in (1, 4, 8, 16):
                if only and (float(only[1]) != sparsity or int(only[2]) != T):
                    continue
                mask = rng.random((T, F)) < prof[None, :]
                a_union = int(mask.any(0).sum())
                idx = torch.from_numpy(np.where(mask, 1.0, -1.0).astype(np.float32)).cuda()
                x = (torch.randn(T, d, device="cuda", generator=gen)).to(torch.float16).float()
                h = torch.relu(torch.randn(T, F, device="cuda", generator=gen)) * torch.from_numpy(mask).cuda()
                ops = {
                    "mul_mat_idx": (lambda c: g.ggml_mul_mat_idx(c[0], x, idx), 1),
                    "axpy": (lambda c: g.ggml_axpy(c[2], h, idx), 1),
                    "sparse_ffn": (lambda c: g.sparse_ffn(c[0], c[1], c[2], x, idx), 3),
                }
                row = {"weights": wname, "sparsity": sparsity, "T": T, "active_union": a_union}
                for name, (fn, n_mats) in ops.items():
                    fn(copies[0]); torch.cuda.synchronize()              # sizes the shared workspace before capture
                    graph = torch.cuda.CUDAGraph()
                    with torch.cuda.graph(graph):
                        for c in copies:
                            fn(c)
                    for _ in range(3):
                        graph.replay()
                    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    torch.cuda.synchronize()
                    e0.record()
                    for _ in range(reps):
                        graph.replay()
                    e1.record()
                    torch.cuda.synchronize()
                    us = e0.elapsed_time(e1) * 1e3 / (reps * n_copies)
                    nbytes = n_mats * a_union * rowb + T * d * 4 + T * F * 4
                    row[name] = {"us": round(us, 2), "GBps": round(nbytes / us / 1e3, 1), "frac_of_measured_peak": round(nbytes / us / 1e3 / peak, 3)}
                    del graph
                table.append(row)
        del copies
        torch.cuda.empty_cache()
    # CPU reference beside it: the reference's own ggml operators, all host threads, batch 1
    cpu = []
    if not args.no_cpu_baseline and not only:
        try:
            from oracle import pio
            ref = pio.Ref()
            nth = physical_cores()
            for wtype, wname in ((synth.F16, "F16"), (synth.Q4_0, "Q4_0")):
                wf = rng.standard_normal((F, d), dtype=np.float32) * np.float32(0.02)
                W = ref.quantize_q4_0(wf) if wtype == synth.Q4_0 else wf.astype(np.float16)
                rowb = 2 * d if wtype == synth.F16 else d // 32 * 18
                xh = rng.standard_normal((1, d), dtype=np.float32)
                for sparsity in (0.5, 0.8, 0.9, 0.95):
                    prof = synth.zipf_profile(F, 1.0 - sparsity)[rng.permutation(F)]
                    m = rng.random((1, F)) < prof[None, :]
                    idxh = np.where(m, 1.0, -1.0).astype(np.float32)
                    hh = np.abs(rng.standard_normal((1, F), dtype=np.float32)) * m
                    ref.mul_mat_idx(wtype, W, F, d, xh, idxh, None, 0.0, nth, 3); t_up = ref.last_time
                    ref.axpy(wtype, W, F, d, hh, idxh, None, 0.0, nth, 3); t_dn = ref.last_time
                    a = int(m.sum())
                    cpu.append({"weights": wname, "sparsity": sparsity, "T": 1, "threads": nth,
                                "mul_mat_idx": {"us": round(t_up * 1e6, 1), "GBps": round(a * rowb / t_up / 1e9, 1)},
                                "axpy": {"us": round(t_dn * 1e6, 1), "GBps": round(a * rowb / t_dn / 1e9, 1)},
                                "sparse_ffn": {"us": round((2 * t_up + t_dn) * 1e6, 1), "GBps": round(3 * a * rowb / (2 * t_up + t_dn) / 1e9, 1)}})
        except Exception as ex:
            cpu = [{"unavailable": str(ex)}]
    head = next((r for r in table if r["weights"] == "F16" and r["sparsity"] == 0.8 and r["T"] == 1), table[0])
    head_cpu = next((r for r in cpu if r.get("weights") == "F16" and r.get("sparsity") == 0.8), None)
    line = {"metric": "sparse_ffn_hbm_GBps", "value": head["sparse_ffn"]["GBps"], "unit": "GB/s", "n_gpus": 1, "steps": reps, "warmup": 3,
            "ms_per_step": head["sparse_ffn"]["us"] / 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "f16 / q4_0 rows, f32 accumulate", "data": "synthetic",
            "config": {"workload": "sparse-ffn-13b: one sparse-FFN layer d 5120 F 13824, headline row = FP16, 80 % sparse, batch 1, whole FFN",
                       "l2": "weights rotate over 12 (F16) / 44 (Q4_0) distinct copies: active rows of consecutive iterations exceed 2 x L2"},
            "roofline": {"bound": "hbm", "achieved": head["sparse_ffn"]["GBps"], "peak": peak, "unit": "GB/s",
                         "frac": head["sparse_ffn"]["frac_of_measured_peak"], "peak_source": f"of {peak_kind}", "traffic": None},
            "cpu_baseline": ({"value": head_cpu["sparse_ffn"]["GBps"], "unit": "GB/s", "cores": head_cpu["threads"], "kind": "reference",
                              "sample": "reference ggml mul_mat_idx x2 + axpy on the same shape and sparsity, batch 1, best of 3"} if head_cpu else None),
            "table": table, "cpu_table": cpu, "env_overrides": pi_env()}
    _emit(line)


# ------------------------------------------------------------------------------------------------ main

def _emit(line: dict):
    """The JSON line is the only thing this program writes to its stdout: see _guard_stdout."""
    sys.stdout.flush()
    if _REAL_STDOUT is not None:
        os.write(_REAL_STDOUT, (json.dumps(line) + "\n").encode())
    else:
        print(json.dumps(line), flush=True)


_REAL_STDOUT = None


def _guard_stdout():
    """Libraries loaded below (NCCL prints its version banner on stdout) must not get between the caller and the one JSON
    line: file descriptor 1 is pointed at stderr for the rest of the run and the line is written to the saved descriptor."""
    global _REAL_STDOUT
    sys.stdout.flush()
    _REAL_STDOUT = os.dup(1)
    os.dup2(2, 1)


def main():
    _guard_stdout()
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--config", default=None)
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--layers", type=int, default=None, help="override the layer count (profiling captures of a small case)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--only", default=None, help="sparse-ffn-13b: one case as WEIGHTS:SPARSITY:T, e.g. F16:0.5:1 (profiling captures)")
    args = ap.parse_args()
    K, W = max(1, args.steps), max(3, args.warmup)

    from powerinfer_b200 import configs
    if args.config == "sparse-ffn-13b":
        if int(os.environ.get("RANK", "0")) == 0:
            sparse_ffn_microbench(args)
        return
    cfg_name = args.config or configs.HEADLINE
    cfg = configs.CONFIGS[cfg_name]
    import dataclasses
    spec = cfg["spec"]
    if args.layers:
        spec = dataclasses.replace(spec, n_layer=args.layers)
    P = cfg["prompt"]
    spec = dataclasses.replace(spec, n_ctx=max(spec.n_ctx, P + W + K + 16))
    T = args.batch
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    metric = "decode_tok_per_s" if T == 1 else f"decode_tok_per_s_batch{T}"
    config = {"workload": f"{cfg_name}: decode after a {P}-token prompt, batch {T}, greedy", "n_layer": spec.n_layer, "d_model": spec.d,
              "n_ff": spec.n_ff, "weights": "Q4_0" if spec.wtype == 2 else "F16", "predictor": f"rank {spec.rank} F16",
              "mean_firing": spec.firing, "parallelism": f"neuron+head sharding x{world}" if world > 1 else "single GPU",
              "l2": "inputs (weights, tens of GB per step) are larger than L2; no flush needed"}

    if args.impl == "reference":
        if rank != 0:
            return
        t0 = time.time()
        steps = []
        try:                                          # the stock decode loop on reduced-layer models of the same layer shape
            loop = cpu_reference_decode(spec)
        except Exception as ex:
            loop = {"unavailable": f"{type(ex).__name__}: {ex}"}
        for _ in range(min(K, 3)):                    # each "step" is one bounded sample (one layer's operators + lm head, extrapolated)
            steps.append(cpu_reference(spec))
            if time.time() - t0 > 150:
                break
        ops_best = max(steps, key=lambda r: r["value"])
        best = loop if "value" in loop else ops_best  # headline: the decode loop (it includes attention, norms, RoPE and the graph overhead)
        best = dict(best, operators_only=ops_best, decode_loop=loop)
        line = {"impl": "reference", "metric": metric, "value": best["value"], "unit": "tok/s", "n_gpus": args.gpus, "steps": len(steps),
                "warmup": 0, "steps_requested": K, "ms_per_step": best["ms_per_token"], "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
                "dtype": "q4_0xq8_0 int8 dot, f32 accumulate" if spec.wtype == 2 else "f16 weights, f32 accumulate",
                "data": "synthetic", "config": config, "cpu_baseline": best,
                "e2e": {"value": best["value"], "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
        _emit(line)
        return

    import numpy as np
    import torch
    import torch.distributed as dist
    from powerinfer_b200 import engine, synth_device

    torch.cuda.set_device(local_rank)
    os.environ.setdefault("NCCL_DEBUG", "WARN")          # keep NCCL's version banner off stdout: the JSON line is the only output
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # refuse before allocating anything when this rank's share of the weights cannot fit the device (the weights are drawn
    # once, then packed into the engine's layout: about twice their size at the peak)
    rb = (lambda cols: cols // 32 * 18) if spec.wtype == 2 else (lambda cols: cols * 2)
    per_layer = (spec.d + 2 * spec.d_kv + spec.d) * rb(spec.d) + 3 * spec.n_ff * rb(spec.d) + 2 * spec.rank * (spec.d + spec.n_ff)
    need = spec.n_layer * per_layer / world * 1.25 + 2 * spec.n_vocab * spec.d * 2
    have = torch.cuda.get_device_properties(local_rank).total_memory
    if need > 0.92 * have:
        raise SystemExit(f"bench.py: {cfg_name} needs about {need / 2**30:.0f} GiB per GPU on {world} GPU(s), the device has "
                         f"{have / 2**30:.0f} GiB: run it with more GPUs (--gpus N under torch.distributed.run)")
    g, layers = synth_device.build_local_model(spec, world, rank, seed=0)
    PB = 32                                           # prompt chunk: tokens of one sequence per step
    eng = engine.DecodeEngine(spec, g, max_batch=max(T, PB), n_ranks=world, rank=rank, local_layers=layers)
    del layers
    if world > 1:
        eng.setup_exchange()

    # ---- prompt: through the engine's chunked prompt path (pi_engine_prefill_host), timed on its own
    prompt = np.random.default_rng(0).integers(0, spec.n_vocab, (T, P))
    eng.prefill([int(v) for v in prompt[0, :PB]], seq=0, pos0=0, want_logits=True)       # warm-up: plain run + capture
    eng.prefill([int(v) for v in prompt[0, :PB]], seq=0, pos0=0, want_logits=False)
    eng.prefill([int(v) for v in prompt[0, :PB]], seq=0, pos0=0, want_logits=True)
    eng.prefill([int(v) for v in prompt[0, :PB]], seq=0, pos0=0, want_logits=False)
    barrier()
    t0 = time.perf_counter()
    start_tokens = []
    for b in range(T):
        _, first = eng.prefill([int(v) for v in prompt[b]], seq=b, pos0=0, want_logits=True)
        start_tokens.append(int(first))
    barrier()
    prompt_s = time.perf_counter() - t0
    if world > 1:
        tp = torch.tensor([prompt_s], dtype=torch.float64, device="cuda")
        dist.all_reduce(tp, op=dist.ReduceOp.MAX)
        prompt_s = float(tp[0])

    def reset(pos0):
        eng.set_inputs_device(start_tokens, [pos0] * T)

    # ---- value: device-resident loop
    reset(P)
    for _ in range(W):
        eng.step_device(T); eng.advance(T)
    eng.stream.synchronize()
    sampler = ClockSampler(local_rank) if rank == 0 else None
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    t_host0 = time.monotonic()
    with torch.cuda.stream(eng.stream):
        torch.cuda.nvtx.range_push("timed_steps")     # lets a profiler pick exactly the timed launches (--nvtx-include "timed_steps/")
        ev0.record()
        for _ in range(K):
            eng.step_device(T); eng.advance(T)
        ev1.record()
        torch.cuda.nvtx.range_pop()
    eng.stream.synchronize()
    t_host1 = time.monotonic()
    barrier()
    ms = ev0.elapsed_time(ev1)
    clocks = sampler.stop(t_host0, t_host1) if sampler else None
    eng.status()
    launches_per_step = eng.launches() + 1

    # ---- e2e: host buffers through the C ABI, every step
    reset(P + W)
    eng.h_tokens[:T] = torch.tensor(start_tokens, dtype=torch.int32)
    eng.h_pos[:T] = P + W
    for _ in range(3):
        eng.decode_host_raw(T)
        eng.h_tokens[:T] = eng.h_argmax[:T]; eng.h_pos[:T] += 1
    barrier()
    greedy_ids = []                                   # sequence 0's greedy continuation (a record of the run: on random weights the stream changes with the GPU count, because the partial vectors are added in another order and neurons at the threshold flip)
    t0 = time.perf_counter()
    for _ in range(K):
        eng.decode_host_raw(T)                        # H2D ids+positions, graph, D2H logits + greedy id, synchronize
        eng.h_tokens[:T] = eng.h_argmax[:T]; eng.h_pos[:T] += 1
        if len(greedy_ids) < 32:
            greedy_ids.append(int(eng.h_argmax[0]))
    barrier()
    e2e_ms = (time.perf_counter() - t0) * 1e3

    if world > 1:
        tt = torch.tensor([ms, e2e_ms], dtype=torch.float64, device="cuda")
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        ms, e2e_ms = float(tt[0]), float(tt[1])

    # ---- per-stage profile over the same kind of steps (events around every launch)
    reset(P + W)
    eng.active_total(reset=True)
    n_prof = min(K, 8)
    stage_ms = {}
    for _ in range(n_prof):
        sm, _ = eng.profile_step(T)
        eng.advance(T)
        for k, v in sm.items():
            stage_ms[k] = stage_ms.get(k, 0.0) + v / n_prof
    active = eng.active_total() / (n_prof * spec.n_layer) * world     # mean active neurons per layer (all ranks)
    # ---- per-kernel durations: each stage's kernels for all layers, back to back (overlapped as inside the step)
    b2b = {}
    for st in ("qkv", "out_proj", "predictor", "up_gate", "down", "sparse_ffn", "lm_head", "norm", "attention", "compact"):
        ms_launch, n_launch = eng.time_stage(T, st)     # the norms of a sharded run carry the exchange (all ranks replay them together)
        if n_launch > 0:
            b2b[st] = (ms_launch * 1e3, n_launch)
    # the stated baseline for the exchange: an NCCL all-reduce of one partial vector (T x d floats), timed alone
    nccl_us = None
    if world > 1:
        buf = torch.zeros(T * spec.d, dtype=torch.float32, device="cuda")
        for _ in range(10):
            dist.all_reduce(buf)
        torch.cuda.synchronize()
        a0, a1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a0.record()
        for _ in range(100):
            dist.all_reduce(buf)
        a1.record()
        torch.cuda.synchronize()
        tt = torch.tensor([a0.elapsed_time(a1) * 10.0], dtype=torch.float64, device="cuda")
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        nccl_us = float(tt[0])

    if rank == 0:
        from powerinfer_b200 import configs as C2
        peak, peak_kind = measured_peaks()
        bytes_tok = C2.bytes_per_token(spec, active)
        ops = {}
        for st in ("qkv", "out_proj", "predictor", "up_gate", "down", "sparse_ffn", "lm_head"):
            if stage_ms.get(st, 0.0) <= 0 or st not in b2b:
                continue
            us_launch, n_launch = b2b[st]
            t_ms = us_launch * n_launch * 1e-3
            gbs = bytes_tok[st] / world / (t_ms * 1e-3) / 1e9
            ops[st] = {"ms_per_step": round(t_ms, 4), "launches_per_step": n_launch, "us_per_launch": round(us_launch, 2),
                       "GBps": round(gbs, 1), "frac_of_measured_peak": round(gbs / peak, 3),
                       "serialised_ms_per_step": round(stage_ms[st], 4)}
        dom = max(ops, key=lambda k: ops[k]["ms_per_step"])
        roofline = {"bound": "hbm", "kernel": {"qkv": "k_gemv_ring_w (dense, QKV rows)", "out_proj": "k_gemv_ring_w (dense, out-proj)",
                                               "predictor": "k_gemv_ring_g + k_gemv_ring_w (dense F16, fc1 + fc2)", "up_gate": "k_gather_rows (gather, up+gate)",
                                               "down": "k_axpy_rows",
                                               "sparse_ffn": "k_ffn_rows (gather over up + gate rows, activation, axpy over down rows: one launch)", "lm_head": "k_gemv_ring_w (dense, lm head)"}[dom],
                    "achieved": ops[dom]["GBps"], "peak": peak, "unit": "GB/s", "frac": round(ops[dom]["GBps"] / peak, 3),
                    "peak_source": f"of {peak_kind}", "launches_per_step": ops[dom]["launches_per_step"],
                    "bytes_per_launch": bytes_tok[dom] / world / ops[dom]["launches_per_step"],
                    "mean_launch_us": ops[dom]["us_per_launch"],
                    "how": "this stage's kernels for every layer, back to back in a CUDA graph as inside a step, CUDA events around 5 replays",
                    "traffic": ncu_traffic(cfg_name).get(dom) if world == 1 else None}
        step_bytes = bytes_tok["total"] / world
        line = {"metric": metric, "value": K * T / (ms * 1e-3), "unit": "tok/s", "n_gpus": world, "steps": K, "warmup": W,
                "ms_per_step": ms / K, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
                "dtype": "q4_0 x q8_0 int8 dot, f32 accumulate" if spec.wtype == 2 else "f16 weights, f32 accumulate",
                "data": "synthetic", "config": config,
                "e2e": {"value": K * T / (e2e_ms * 1e-3), "unit": "tok/s", "h2d_bytes_per_step": 8 * T,
                        "d2h_bytes_per_step": T * spec.n_vocab * 4 + 4 * T},
                "gpu_launches": launches_per_step * K, "clocks": clocks, "roofline": roofline,
                "step_hbm": {"algorithmic_GB_per_step_per_gpu": round(step_bytes / 1e9, 3),
                             "GBps": round(step_bytes / (ms / K * 1e-3) / 1e9, 1),
                             "frac_of_measured_peak": round(step_bytes / (ms / K * 1e-3) / 1e9 / peak, 3)},
                "ops": ops, "latency_stages": {st: {"ms_per_step": round(b2b[st][0] * b2b[st][1] * 1e-3, 4), "launches_per_step": b2b[st][1],
                                                    "us_per_launch": round(b2b[st][0], 2)} for st in ("norm", "attention", "compact") if st in b2b},
                "exchange": ({"kernel": "inside the norm that consumes the sum (k_norm_cluster): each value stored into the peers beside the number of the exchange, bounded poll, no flag and no fence",
                              "per_step": spec.n_layer * (1 if spec.arch == 1 else 2), "bytes_per_exchange_per_peer": T * spec.d * 4,
                              "nccl_all_reduce_same_bytes_us": round(nccl_us, 2)} if world > 1 else None),
                "greedy_ids": greedy_ids,
                "prompt_tok_per_s": round(T * P / prompt_s, 1), "prompt_chunk": PB,
                "stage_ms_profiled": {k: round(v, 4) for k, v in stage_ms.items()},
                "mean_active_neurons_per_layer": round(active, 1), "env_overrides": pi_env()}
        if world == 1 and not args.no_cpu_baseline:
            try:
                line["cpu_baseline"] = cpu_reference(spec)
            except Exception as ex:                     # the checker is optional at run time; say so rather than fail the bench
                line["cpu_baseline"] = {"value": None, "unit": "tok/s", "cores": 0, "kind": "reference", "sample": f"unavailable: {ex}"}
        _emit(line)
    eng.close()
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
