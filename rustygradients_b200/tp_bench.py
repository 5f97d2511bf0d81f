"""Tensor-parallel token loop: microseconds per token with the one-shot peer-memory
all-reduce and with NCCL, on the GPT-2-XL shape (vocabulary 50257, d_model 1600,
25 heads, bf16 weights), one process per GPU.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P \\
        -m rustygradients_b200.tp_bench [--layers 48] [--batch 1] [--prompt 512] [--steps 64]

Rank 0 prints one JSON line.  Weights are seeded random; both modes run the same steps
from the same cached prompt and their ids are compared."""
from __future__ import annotations

import argparse
import json
import os

import numpy as np


def main() -> None:
    import torch
    import torch.distributed as dist

    from . import B200Backend, GptConfig, GPTModel

    ap = argparse.ArgumentParser()
    ap.add_argument("--layers", type=int, default=48)
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--prompt", type=int, default=512)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--d-model", type=int, default=1600)
    ap.add_argument("--heads", type=int, default=25)
    ap.add_argument("--vocab", type=int, default=50257)
    a = ap.parse_args()
    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", str(rank)))
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29533")
    dist.init_process_group("gloo", rank=rank, world_size=world)  # host channel: the 128-byte id and the timing max
    torch.cuda.set_device(local)
    be = B200Backend(local)
    stream = torch.cuda.ExternalStream(be.stream, device=torch.device("cuda", local))
    cfg = GptConfig(1024, a.vocab, a.layers, a.heads, a.d_model, weight_dtype="bf16", max_batch=a.batch,
                    tp_rank=rank, tp_size=world)
    rng = np.random.Generator(np.random.PCG64(5))
    prompt = rng.integers(0, a.vocab, size=(a.batch, a.prompt), dtype=np.uint32)
    out = {}
    ids = {}
    params = None
    for mode in ("peer", "nccl"):
        os.environ["RG_B200_TP_ALLREDUCE"] = mode
        m = GPTModel(be, cfg)
        if params is None:
            prng = np.random.Generator(np.random.PCG64(6))
            params = [(prng.standard_normal(s, dtype=np.float32) * np.float32(0.02)) if s[0] != 1 or s[1] == a.vocab
                      else np.ones(s, np.float32) for s in m.parameter_shapes()]
        m.load_parameters(params)
        if world > 1:
            ident = [GPTModel.tp_unique_id() if rank == 0 else None]
            dist.broadcast_object_list(ident, src=0)
            m.tp_init(ident[0])
        fused = m.tp_fused()
        m.prefill(prompt, want_logits=False)
        m.decode_run(8)  # warm-up (graph capture)
        m.rewind(a.prompt)
        be.synchronize()
        dist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        m.decode_run(a.steps)
        e1.record(stream)
        be.synchronize()
        t = torch.tensor([e0.elapsed_time(e1)], dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ids[mode] = m.read_tokens(a.prompt, a.steps, a.batch)
        out[mode] = {"fused": fused, "us_per_token": float(t.item()) * 1e3 / a.steps,
                     "tokens_per_s": a.batch * a.steps / (float(t.item()) * 1e-3)}
        bytes_step = m.decode_step_bytes(a.batch, a.prompt + a.steps / 2)
        out[mode]["algorithmic_gb_per_s_per_gpu"] = bytes_step / (float(t.item()) * 1e-3 / a.steps) / 1e9
        m.close()
        dist.barrier()
    if rank == 0:
        same = float((ids["peer"] == ids["nccl"]).mean())
        print(json.dumps({"workload": f"d_model {a.d_model}, {a.layers} layers, {a.heads} heads, vocab {a.vocab}, bf16, batch "
                                      f"{a.batch}, prompt {a.prompt}, {a.steps} steps", "tp_size": world, **out,
                          "ids_equal_fraction": same}))
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
