#!/usr/bin/env python
"""Benchmark of the GPT token loop: decode tokens/sec on the GPT-2-small shape
(vocab 1024, d_model 768, 12 layers, 12 heads, context 1024, f32 weights, batch 1
per GPU, prompt 128 ids, greedy decode of 256 ids) and its fraction of the HBM
roofline.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

One "step" is one decode run: the 256 token-loop iterations that follow a
128-id prompt whose keys/values are already in the cache (positions 128..383).
`value` times K such steps with everything resident in HBM; `e2e` times the
public generate() call with host buffers (prompt upload, prompt pass, decode,
ids download).  With N > 1 (under torchrun) every rank runs its own sequence on
its own GPU: sequences are the shard, there is no collective in the loop.

Two more records ride in the same JSON line (skipped with --no-extra):
  "batched": the GPT-2-small shape with the full vocabulary and bf16 weights, prompt 256, decode 256, 64 sequences
             in total split over the N ranks (strong scaling) and 64 sequences on every rank (weak scaling);
  "tp":      (N >= 2) the GPT-2-XL shape, bf16, prompt 512, decode 256, tensor parallel over the N ranks with the
             peer-memory all-reduce, batch 1 and batch 32, bytes counted PER GPU.
Prints ONE JSON line on rank 0.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

WORKLOAD = "gpt2-small-shape vocab1024 f32 batch1 prompt128 decode256"
CFG_INDEX = 1
EXTRAS_BUDGET_S = 360          # time the extra records may take before the headline is printed without them
NOMINAL_HBM_GBS = 8000.0     # the figure the metric's roofline is defined on
FALLBACK_HBM_GBS = 6650.0
NCU_TRAFFIC_RATIO = 1.0036   # measured DRAM bytes (read + write) / algorithmic bytes, profiles/token_loop_kernel_*


def measured_hbm_peak():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(p) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return FALLBACK_HBM_GBS, "fallback"


# --------------------------------------------------------------------------
# clocks: sampled DURING the timed region
# --------------------------------------------------------------------------
class ClockSampler:
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu = gpu_index
        self.rows = []
        self.proc = None
        self.thread = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.gpu}", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except Exception:
            self.proc = None
            return
        self.thread = threading.Thread(target=self._read, daemon=True)
        self.thread.start()

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append((time.time(), [c.strip() for c in line.split(",")]))

    def stop(self, t0: float, t1: float):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        rows = [r for t, r in self.rows if t0 - 0.05 <= t <= t1 + 0.15] or [r for _, r in self.rows]
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in rows:
            try:
                sm.append(float(r[0]))
                mx.append(float(r[1]))
            except Exception:
                continue
            for name, val in zip(names, r[3:7]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


# --------------------------------------------------------------------------
# the CPU arm: the reference's own algorithm (full re-forward of the whole
# context for every new id, no KV cache, unmasked attention, ReLU, all T logit
# rows) restated in numpy f32 over the bundled OpenBLAS, on the host cores.
# --------------------------------------------------------------------------
def cpu_threads() -> int:
    try:
        from threadpoolctl import threadpool_info
        n = [i.get("num_threads", 0) for i in threadpool_info() if i.get("user_api") == "blas"]
        if n:
            return int(max(n))
    except Exception:
        pass
    return os.cpu_count() or 1


def use_all_host_threads() -> None:
    """torchrun exports OMP_NUM_THREADS=1; the CPU arm is meant to use every host core."""
    try:
        from threadpoolctl import threadpool_limits
        threadpool_limits(limits=os.cpu_count() or 1, user_api="blas")
    except Exception:
        pass


def cpu_reference_tokens_per_s(n_tokens: int, params=None):
    """Times n_tokens iterations of the reference loop at context lengths spread
    evenly over the workload's 128..383 range; returns (tokens/s, seconds)."""
    from oracle import gpt_oracle as O
    use_all_host_threads()
    c = O.CONFIGS[CFG_INDEX]
    cfg, P, G = c["cfg"], c["prompt"], c["gen"]
    seed = O.config_seed(CFG_INDEX)
    if params is None:
        params = O.make_params(cfg, seed)
    rng = np.random.Generator(np.random.PCG64(seed + 1))
    ctxs = np.linspace(P, P + G - 1, n_tokens).round().astype(int)
    ids = rng.integers(0, cfg.vocab_size, size=(1, P + G), dtype=np.int64)
    O.forward(params, cfg, ids[:, :P], causal=False, act="relu")  # warm the BLAS threads
    t0 = time.perf_counter()
    for T in ctxs:
        lg = O.forward(params, cfg, ids[:, :T], causal=False, act="relu")   # all T rows, like gpt.rs:79-80
        O.greedy_pick(lg[0, -1])
    dt = time.perf_counter() - t0
    return n_tokens / dt, dt


def run_reference(args, rank: int) -> None:
    if rank != 0:
        return
    sample = 6
    for _ in range(args.warmup):
        pass  # warm-up is the BLAS warm call inside cpu_reference_tokens_per_s
    from oracle import gpt_oracle as O
    params = O.make_params(O.CONFIGS[CFG_INDEX]["cfg"], O.config_seed(CFG_INDEX))
    t_all, n_all = 0.0, 0
    for _ in range(args.steps):
        _, dt = cpu_reference_tokens_per_s(sample, params)
        t_all += dt
        n_all += sample
    v = n_all / t_all
    cores = cpu_threads()
    desc = (f"{sample} loop iterations per step at context lengths spread over 128..383, full re-forward per id "
            f"(no KV cache, unmasked attention, ReLU, all logit rows), numpy f32 + OpenBLAS")
    line = {"impl": "reference", "metric": "decode tokens/sec (GPT-2-small shape)", "value": v, "unit": "tokens/s",
            "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * t_all / args.steps,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": WORKLOAD, "kv_cache": False, "causal": False, "activation": "relu"},
            "cpu_baseline": {"value": v, "unit": "tokens/s", "cores": cores, "kind": "port", "sample": desc},
            "e2e": {"value": v, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line), flush=True)


# --------------------------------------------------------------------------
# the sharded batch and the tensor-parallel model (records inside the main line)
# --------------------------------------------------------------------------
def _timed_decode(torch, model, be, stream, barrier, P, G, runs):
    """ms per decode run of G steps from position P (device time, this rank); one untimed run first."""
    model.rewind(P)
    model.decode_run(G)
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for _ in range(runs):
        model.rewind(P)
        model.decode_run(G)
    e1.record(stream)
    be.synchronize()
    barrier()
    return e0.elapsed_time(e1) / runs


def _sum_over_ranks(torch, value, world, dev):
    if world == 1:
        return int(value)
    import torch.distributed as dist
    t = torch.tensor([int(value)], dtype=torch.int64, device=dev)
    dist.all_reduce(t)
    return int(t.item())


def run_batched(torch, rg, O, be, dev, stream, barrier, rank, world):
    """Configuration 2 of the oracle's list: vocabulary 50257, bf16 weights, prompt 256, decode 256; 64 sequences."""
    from rustygradients_b200.sharding import max_over_ranks, shard_range
    c = O.CONFIGS[2]
    cfg, P, G, TOTAL = c["cfg"], c["prompt"], c["gen"], 64
    seed = O.config_seed(2)
    params = O.make_params(cfg, seed)                 # f32 draws; the engine rounds them to bf16 (RNE) at load
    model = rg.GPTModel(be, rg.GptConfig(cfg.block_size, cfg.vocab_size, cfg.num_layers, cfg.num_heads, cfg.embedding_dim,
                                         weight_dtype="bf16", max_batch=TOTAL))
    model.load_parameters(params)
    peak, _ = measured_hbm_peak()
    mean_ctx = P + (G - 1) / 2.0 + 1.0
    rec = {"workload": f"gpt2-small-shape vocab50257 bf16 prompt{P} decode{G}, {TOTAL} sequences", "kv_cache": "bf16"}
    prompts = O.make_prompt(cfg, seed, TOTAL * world, P)
    legs = [("strong", shard_range(TOTAL, rank, world))]
    if world > 1:
        legs.append(("weak", (rank * TOTAL, (rank + 1) * TOTAL)))
    for name, (lo, hi) in legs:
        B = hi - lo
        model.prefill(np.ascontiguousarray(prompts[lo:hi]), want_logits=False)
        ms = max_over_ranks(_timed_decode(torch, model, be, stream, barrier, P, G, 3), world, dev)
        ids = model.read_tokens(P + 1, G - 1, B)
        n_seq = TOTAL if name == "strong" else TOTAL * world
        step_bytes = model.decode_step_bytes(B, mean_ctx)         # this GPU, one token step
        gbs = step_bytes / (ms * 1e-3 / G) / 1e9
        rec[name] = {"sequences_total": n_seq, "sequences_per_gpu": B, "tokens_per_s": n_seq * G / (ms * 1e-3),
                     "us_per_step": ms * 1e3 / G, "bytes_per_step_per_gpu": step_bytes, "gb_per_s_per_gpu": gbs,
                     "frac_of_measured_peak": gbs / peak, "frac_of_8TBs_nominal": gbs / NOMINAL_HBM_GBS,
                     "ids_checksum": _sum_over_ranks(torch, np.asarray(ids, dtype=np.uint64).sum(), world, dev)}
    if world == 1:
        rec["weak"] = rec["strong"]
    model.close()
    return rec


def _pooled_params(shapes, vocab, seed):
    """Synthetic weights for a large model without drawing 1.5 G normals per rank: one pool of N(0, 0.02) values, every
    tensor a window of it at its own offset (zero-copy views; vectors of shape [1, n] are ones, the LM-head bias excepted,
    as in the draw this replaces).  Every rank builds the same list from the same seed and keeps its shard of it."""
    sizes = [int(s[0]) * int(s[1]) for s in shapes]
    pool_n = max(sizes) + (1 << 22)
    pool = np.random.Generator(np.random.PCG64(seed)).standard_normal(pool_n, dtype=np.float32) * np.float32(0.02)
    out, off = [], 0
    for i, (s, n) in enumerate(zip(shapes, sizes)):
        if s[0] != 1 or s[1] == vocab:
            off = (off + 1000003 * (i + 1)) % (pool_n - n + 1)
            out.append(pool[off:off + n].reshape(s))
        else:
            out.append(np.ones(s, np.float32))
    return out


def run_tp(torch, rg, be, dev, stream, barrier, rank, world):
    """GPT-2-XL shape (vocabulary 50257, d_model 1600, 48 layers, 25 heads), bf16, tensor parallel over all ranks."""
    import torch.distributed as dist
    from rustygradients_b200.sharding import max_over_ranks
    V, D, L, H, P, G = 50257, 1600, 48, 25, 512, 256
    peak, _ = measured_hbm_peak()
    model = rg.GPTModel(be, rg.GptConfig(1024, V, L, H, D, weight_dtype="bf16", max_batch=32, tp_rank=rank, tp_size=world))
    model.load_parameters(_pooled_params(model.parameter_shapes(), V, 20245))   # every rank keeps its shard of the same list
    ident = torch.zeros(128, dtype=torch.uint8, device=dev)
    if rank == 0:
        ident = torch.tensor(list(rg.GPTModel.tp_unique_id()), dtype=torch.uint8, device=dev)
    dist.broadcast(ident, src=0)
    model.tp_init(bytes(ident.cpu().tolist()))
    rec = {"workload": f"gpt2-xl-shape vocab{V} bf16 prompt{P} decode{G}", "tp_size": world,
           "allreduce": "peer-memory kernel" if model.tp_fused() else "nccl"}
    rng = np.random.Generator(np.random.PCG64(20246))
    for B in (1, 32):
        prompt = rng.integers(0, V, size=(B, P), dtype=np.uint32)
        model.prefill(prompt, want_logits=False)
        ms = max_over_ranks(_timed_decode(torch, model, be, stream, barrier, P, G, 2), world, dev)
        ids = model.read_tokens(P + 1, G - 1, B)
        step_bytes = model.decode_step_bytes(B, P + (G - 1) / 2.0 + 1.0)     # per GPU: the sharded terms divided by tp_size
        gbs = step_bytes / (ms * 1e-3 / G) / 1e9
        rec[f"batch{B}"] = {"tokens_per_s": B * G / (ms * 1e-3), "us_per_step": ms * 1e3 / G,
                            "bytes_per_step_per_gpu": step_bytes, "gb_per_s_per_gpu": gbs,
                            "frac_of_measured_peak": gbs / peak, "frac_of_8TBs_nominal": gbs / NOMINAL_HBM_GBS,
                            "ids_checksum": int(np.asarray(ids, dtype=np.uint64).sum())}
    model.close()
    return rec


# --------------------------------------------------------------------------
# our arm
# --------------------------------------------------------------------------
def run_ours(args, rank: int, local_rank: int, world: int) -> None:
    import torch
    import rustygradients_b200 as rg
    from oracle import gpt_oracle as O   # seeded weights / prompt generator and the CPU-baseline leg only
    from rustygradients_b200.sharding import gather_ids, max_over_ranks, shard_range

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a B200: there is no CPU fallback for the product path")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)

    c = O.CONFIGS[CFG_INDEX]
    cfg, P, G = c["cfg"], c["prompt"], c["gen"]
    if args.tokens_per_step:
        G = args.tokens_per_step
    seed = O.config_seed(CFG_INDEX)
    B = 1                                   # sequences per GPU (weak scaling: world sequences in total)
    lo, hi = shard_range(world * B, rank, world)
    params = O.make_params(cfg, seed)       # every rank holds a full replica of the same weights
    prompts_all = O.make_prompt(cfg, seed, world * B, P)
    prompt = np.ascontiguousarray(prompts_all[lo:hi])

    be = rg.B200Backend(local_rank)
    model = rg.GPTModel(be, rg.GptConfig(cfg.block_size, cfg.vocab_size, cfg.num_layers, cfg.num_heads,
                                         cfg.embedding_dim, causal=True, activation="gelu_tanh", weight_dtype="f32",
                                         max_batch=B))
    model.load_parameters(params)
    stream = torch.cuda.ExternalStream(be.stream, device=dev)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(dev)

    # ---- device-resident decode: prompt keys/values cached once, then K runs of G token steps
    model.prefill(prompt, want_logits=False)
    first_pick = model.read_tokens(P, 1, B)          # the id the prompt pass chose; fed at position P
    for _ in range(args.warmup):
        model.rewind(P)
        model.decode_run(G)
    barrier()
    sampler = ClockSampler(local_rank)
    sampler.start()
    time.sleep(0.25)
    l0 = be.launch_count
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    t_wall0 = time.time()
    ev0.record(stream)
    for _ in range(args.steps):
        model.rewind(P)
        model.decode_run(G)
    ev1.record(stream)
    be.synchronize()
    barrier()
    t_wall1 = time.time()
    launches = be.launch_count - l0
    ms = max_over_ranks(ev0.elapsed_time(ev1), world, dev)
    clocks = sampler.stop(t_wall0, t_wall1)
    ids_dev = model.read_tokens(P + 1, G - 1, B)       # picks of steps 0..G-2 (the last has no slot to keep)
    step_bytes_main = model.decode_step_bytes(B, P + (G - 1) / 2.0 + 1.0)

    # ---- end to end through the public generate(): host prompt in, host ids out
    pin_prompt = torch.from_numpy(prompt.astype(np.int64)).to(torch.int32).pin_memory()
    prompt_pinned = pin_prompt.numpy().view(np.uint32)
    for _ in range(min(args.warmup, 3)):
        model.generate(prompt_pinned, G)
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    n_e2e = max(3, min(args.steps, 10))
    e0.record(stream)
    for _ in range(n_e2e):
        ids_e2e = model.generate(prompt_pinned, G)
    e1.record(stream)
    be.synchronize()
    barrier()
    ms_e2e = max_over_ranks(e0.elapsed_time(e1), world, dev)
    assert np.array_equal(ids_e2e[:, 1:], ids_dev), "generate() and the device-resident loop disagree"
    assert int(first_pick[0, 0]) == int(ids_e2e[0, 0])
    all_ids = gather_ids(ids_e2e, world * B, rank, world, dev)   # once, after the loop: the only exchange
    model.close()
    line = None
    if rank == 0:
        tokens = world * B * G * args.steps
        value = tokens / (ms * 1e-3)
        e2e_value = world * B * G * n_e2e / (ms_e2e * 1e-3)
        mean_ctx = P + (G - 1) / 2.0 + 1.0              # keys visible to a step, averaged over the run
        step_bytes = step_bytes_main                        # one GPU, one token step
        t_step = ms * 1e-3 / (args.steps * G)               # seconds per token step (slowest rank)
        achieved = step_bytes / t_step / 1e9
        peak, peak_kind = measured_hbm_peak()
        line = {
            "metric": "decode tokens/sec (GPT-2-small shape)", "value": value, "unit": "tokens/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms / args.steps, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": WORKLOAD if G == c["gen"] else WORKLOAD + f" (SHORTENED to {G} tokens: not a bench value)",
                       "sequences_per_gpu": B, "tokens_per_step": G, "kv_cache": "f32", "causal": True,
                       "activation": "gelu_tanh",
                       "l2": "inputs larger than L2 (343 MB of weights streamed per token vs 126 MB L2)",
                       "parallelism": f"{world} independent sequence shard(s), no collective in the loop"},
            "us_per_token": t_step * 1e6,
            "roofline": {"bound": "hbm",
                         "kernel": ((("rg_cluster_loop_kernel" if os.environ.get("RG_B200_DECODE") == "cluster" else "rg_token_loop_kernel")
                                     + f": one persistent cooperative launch per step ({G} token-loop iterations)")
                                    if launches <= 2 * args.steps else
                                    f"token step = {launches // (args.steps * G)} kernels replayed as one CUDA graph"),
                         "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                         "peak_kind": peak_kind, "bytes_per_launch": step_bytes * G,
                         "bytes_per_token": step_bytes, "launch_ms": ms / args.steps,
                         "frac_of_8TBs_nominal": achieved / NOMINAL_HBM_GBS,
                         # dram__bytes_read+write of one ncu capture of the same kernel on 8 tokens (354.4 MB per token
                         # against 353.1 MB algorithmic at that context), scaled to this launch by the tokens it runs
                         "traffic": step_bytes * G * NCU_TRAFFIC_RATIO if launches <= 2 * args.steps else None,
                         "traffic_source": "not measured in this run: algorithmic bytes x 1.0036, the DRAM read+write ratio of "
                                           "the ncu capture in profiles/token_loop_kernel_gpt2small_ncu_full.md"},
            "e2e": {"value": e2e_value, "unit": "tokens/s", "h2d_bytes_per_step": int(B * P * 4),
                    "d2h_bytes_per_step": int(B * G * 4), "calls": n_e2e,
                    "what": "generate(prompt, 256): pinned host ids -> device, prompt pass, 255 cached steps, ids -> host"},
            "gpu_launches": int(launches), "clocks": clocks,
            "ids_checksum": int(np.asarray(all_ids, dtype=np.uint64).sum()),
        }
        if world == 1 and not args.no_cpu_baseline:     # host cores only: timed before the extra records use the GPU again
            v, dt = cpu_reference_tokens_per_s(24, params)
            line["cpu_baseline"] = {
                "value": v, "unit": "tokens/s", "cores": cpu_threads(), "kind": "port", "causal": False,
                "activation": "relu", "kv_cache": False,
                "sample": f"24 loop iterations at context lengths spread over 128..383 ({dt:.1f} s): the reference's loop "
                          "(full re-forward per id, no KV cache, unmasked attention, ReLU, all logit rows) in numpy f32 + OpenBLAS"}
    # ---- extra records (batched, tensor parallel).  The headline above is complete; whatever happens below, it is
    # printed: a failure that every rank sees is reported inside the record, and if the extras do not finish within
    # their time budget (a rank stuck in a collective, say) every rank's watchdog ends its process after rank 0 has
    # printed the line with what was finished until then.
    extra = {}
    extras_done = threading.Event()

    def _watchdog():
        if extras_done.wait(EXTRAS_BUDGET_S):
            return
        if rank == 0:
            out = dict(line)
            out.update(extra)
            for key in (("batched", "tp") if world > 1 else ("batched",)):
                out.setdefault(key, {"error": f"did not finish within {EXTRAS_BUDGET_S} s; the process was ended"})
            print(json.dumps(out), flush=True)
        os._exit(0)

    if not args.no_extra:
        threading.Thread(target=_watchdog, daemon=True).start()
        try:
            extra["batched"] = run_batched(torch, rg, O, be, dev, stream, barrier, rank, world)
        except Exception as e:  # noqa: BLE001  (library errors and torch / NCCL errors alike: the headline is printed either way)
            extra["batched"] = {"error": f"{type(e).__name__}: {e}"}
        if world > 1:
            try:
                extra["tp"] = run_tp(torch, rg, be, dev, stream, barrier, rank, world)
            except Exception as e:  # noqa: BLE001  (library errors and torch / NCCL errors alike: the headline is printed either way)
                extra["tp"] = {"error": f"{type(e).__name__}: {e}"}
        extras_done.set()

    if rank == 0:
        line.update(extra)
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


# --------------------------------------------------------------------------
# single small workloads for profiler captures: python bench.py --only decode|prefill|ingest [...]
# (and, under torchrun, --only tptrace: device trace of the tensor-parallel token loop)
# (not the benchmark: they print their own JSON line and leave the contract line alone)
# --------------------------------------------------------------------------
def _random_params(model, vocab, seed):
    rng = np.random.Generator(np.random.PCG64(seed))
    return [(rng.standard_normal(s, dtype=np.float32) * np.float32(0.02)) if s[0] != 1 or s[1] == vocab
            else np.ones(s, np.float32) for s in model.parameter_shapes()]


def run_tp_trace(a) -> None:
    """Under torchrun: the GPT-2-XL-shape tensor-parallel model of run_tp(), one sequence, and the persistent kernel's
    own time stamps of the middle block of the last token (rank 0 prints them): per stage, median and latest CTA."""
    import torch
    import torch.distributed as dist
    import rustygradients_b200 as rg
    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    if world < 2:
        raise SystemExit("--only tptrace runs under torchrun with 2 or more ranks")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", device_id=dev)
    be = rg.B200Backend(rank)
    V, D, L, H, P, G = 50257, 1600, 48, 25, 512, 64
    model = rg.GPTModel(be, rg.GptConfig(1024, V, L, H, D, weight_dtype="bf16", max_batch=4, tp_rank=rank, tp_size=world))
    model.load_parameters(_pooled_params(model.parameter_shapes(), V, 20245))
    ident = torch.zeros(128, dtype=torch.uint8, device=dev)
    if rank == 0:
        ident = torch.tensor(list(rg.GPTModel.tp_unique_id()), dtype=torch.uint8, device=dev)
    dist.broadcast(ident, src=0)
    model.tp_init(bytes(ident.cpu().tolist()))
    prompt = np.random.Generator(np.random.PCG64(20246)).integers(0, V, size=(1, P), dtype=np.uint32)
    model.prefill(prompt, want_logits=False)
    for _ in range(2):
        model.rewind(P)
        model.decode_run(G)
    be.synchronize()
    dist.barrier()
    t = time.perf_counter()
    model.rewind(P)
    model.decode_run(G)
    be.synchronize()
    us = (time.perf_counter() - t) / G * 1e6
    model.trace(True)
    model.rewind(P)
    model.decode_run(G)
    be.synchronize()
    tr = model.read_trace(1 << 17).astype(np.int64)
    if rank == 0:
        ok = tr[:, 4] > 0
        blk = L // 2
        t0 = tr[ok & (tr[:, 3] == blk)][:, 4].min()
        stages = {}
        for st, name in enumerate(("qkv", "attention", "out_projection", "fc1", "fc2")):
            sel = tr[ok & (tr[:, 3] == blk) & (tr[:, 2] == st)]
            if len(sel):
                r = (sel[:, 4:8] - t0) / 1e3
                stages[name] = {"ctas": int(len(sel)),
                                "median_us": [round(float(np.median(r[:, i])), 2) for i in range(4)],
                                "latest_us": [round(float(r[:, i].max()), 2) for i in range(4)]}
        first = tr[ok & (tr[:, 2] == 0)]
        starts = [np.median(first[first[:, 3] == l][:, 4]) for l in range(L)]
        print(json.dumps({"only": "tptrace", "tp_size": world, "us_per_token": us, "block": blk,
                          "columns": ["start", "input ready", "dot products done", "outputs stored"], "stages": stages,
                          "block_period_us": round(float(np.median(np.diff(starts))) / 1e3, 2)}))
    dist.barrier()
    model.close()
    dist.destroy_process_group()


def run_only(a) -> None:
    import torch
    import rustygradients_b200 as rg
    be = rg.B200Backend(0)
    stream = torch.cuda.ExternalStream(be.stream, device=torch.device("cuda", 0))
    rng = np.random.Generator(np.random.PCG64(9))
    D, H, L, V = a.d_model, a.heads, a.layers, a.vocab
    if a.only == "decode":
        # token-step time of `batch` sequences: batches 1, 2, 4 run in the persistent kernel, larger ones as separate launches
        m = rg.GPTModel(be, rg.GptConfig(1024, V, L, H, D, weight_dtype=a.dtype, max_batch=a.batch))
        m.load_parameters(_random_params(m, V, 9))
        prompt = rng.integers(0, V, size=(a.batch, a.prompt), dtype=np.uint32)
        m.prefill(prompt, want_logits=False)
        m.decode_run(min(a.iters, 40))
        times = []
        for _ in range(3):
            m.rewind(a.prompt)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(stream)
            m.decode_run(a.iters)
            e1.record(stream)
            be.synchronize()
            times.append(e0.elapsed_time(e1) * 1e3 / a.iters)
        us = min(times)
        by = m.decode_step_bytes(a.batch, a.prompt + a.iters / 2)
        print(json.dumps({"only": "decode", "batch": a.batch, "dtype": a.dtype, "prompt": a.prompt, "steps": a.iters,
                          "us_per_step": us, "tokens_per_s": a.batch / (us * 1e-6),
                          "algorithmic_gb_per_s": by / (us * 1e-6) / 1e9, "launches": be.launch_count}))
    elif a.only == "prefill":
        # prompt pass of `batch` prompts (the tensor-core part of the path); RG_B200_PREFILL=simt times the CUDA-core GEMM
        m = rg.GPTModel(be, rg.GptConfig(1024, V, L, H, D, weight_dtype=a.dtype, max_batch=a.batch))
        m.load_parameters(_random_params(m, V, 7))
        ids = rng.integers(0, V, size=(a.batch, a.prompt), dtype=np.uint32)
        m.prefill(ids, want_logits=False)
        be.synchronize()
        t0 = time.perf_counter()
        for _ in range(a.iters):
            m.prefill(ids, want_logits=False)
        be.synchronize()
        dt = (time.perf_counter() - t0) / a.iters
        rows = a.batch * a.prompt
        flops = 2.0 * rows * L * 12 * D * D + 2.0 * a.batch * D * V + 4.0 * L * a.batch * a.prompt * a.prompt * D / 2
        print(json.dumps({"only": "prefill", "prompt_pass_ms": dt * 1e3, "tflops": flops / dt / 1e12, "rows": rows, "layers": L,
                          "gemm": os.environ.get("RG_B200_PREFILL", "tcgen05"), "launches": be.launch_count}))
    else:
        # time from a safetensors file on disk (page cache) to a model that is ready to generate
        from rustygradients_b200 import serialization as S
        C = 1024

        def n(*shape):
            return rng.standard_normal(shape, dtype=np.float32) * np.float32(0.02)

        t = {}
        m = rg.GPTModel(be, rg.GptConfig(C, V, L, H, D))
        if a.names == "hf_gpt2":
            t["wte.weight"], t["wpe.weight"] = n(V, D), n(C, D)
            for l in range(L):
                h = f"h.{l}."
                t[h + "attn.c_attn.weight"], t[h + "attn.c_attn.bias"] = n(D, 3 * D), n(3 * D)
                t[h + "attn.c_proj.weight"], t[h + "attn.c_proj.bias"] = n(D, D), n(D)
                t[h + "mlp.c_fc.weight"], t[h + "mlp.c_fc.bias"] = n(D, 4 * D), n(4 * D)
                t[h + "mlp.c_proj.weight"], t[h + "mlp.c_proj.bias"] = n(4 * D, D), n(D)
                for ln in ("ln_1", "ln_2"):
                    t[h + ln + ".weight"], t[h + ln + ".bias"] = np.ones(D, np.float32), np.zeros(D, np.float32)
            t["ln_f.weight"], t["ln_f.bias"] = np.ones(D, np.float32), np.zeros(D, np.float32)
        else:
            for name, shp in zip(S.rusty_names(L), m.parameter_shapes()):
                t[name] = n(*shp)
        path = os.path.join("/tmp", f"rg_ingest_bench_{os.getpid()}.safetensors")
        S.write_safetensors(path, t)
        size = os.path.getsize(path)
        del t
        try:
            times = []
            for _ in range(3):
                be.synchronize()
                t0 = time.perf_counter()
                m.load_safetensors(path, names=a.names)
                be.synchronize()
                times.append(time.perf_counter() - t0)
            ids = m.generate(np.zeros((1, 4), np.uint32), 4)
            print(json.dumps({"only": "ingest", "file_bytes": size, "names": a.names, "load_s": times,
                              "best_gb_per_s": size / min(times) / 1e9, "generated": [int(x) for x in np.asarray(ids).ravel()]}))
        finally:
            os.remove(path)


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-extra", action="store_true", help="skip the batched and tensor-parallel records")
    ap.add_argument("--tokens-per-step", type=int, default=0,
                    help="shorten the decode run (profiling only; the default is the workload's 256)")
    ap.add_argument("--only", choices=["decode", "prefill", "ingest", "tptrace"],
                    help="run one small workload for a profiler capture instead of the benchmark")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--prompt", type=int, default=256)
    ap.add_argument("--layers", type=int, default=12)
    ap.add_argument("--iters", type=int, default=3, help="--only: timed repetitions (decode: token steps)")
    ap.add_argument("--dtype", default="bf16", choices=["bf16", "f32"])
    ap.add_argument("--vocab", type=int, default=50257)
    ap.add_argument("--d-model", type=int, default=768)
    ap.add_argument("--heads", type=int, default=12)
    ap.add_argument("--names", default="hf_gpt2", choices=["hf_gpt2", "rusty"])
    args = ap.parse_args()
    if args.only == "tptrace":
        run_tp_trace(args)
        return
    if args.only:
        run_only(args)
        return
    args.warmup = max(3, args.warmup) if args.impl == "ours" else args.warmup
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if args.impl == "reference":
        run_reference(args, rank)
        return
    if world != args.gpus:
        if args.gpus == 1 and world == 1:
            pass
        else:
            raise SystemExit(f"--gpus {args.gpus} needs torchrun with {args.gpus} ranks (WORLD_SIZE={world})")
    run_ours(args, rank, local_rank, world)


if __name__ == "__main__":
    main()
