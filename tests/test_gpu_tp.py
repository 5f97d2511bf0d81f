"""Tensor-parallel token loop on 2 GPUs against the oracle (and so against the
single-GPU path, which the other tests tie to the oracle).  Needs two GPUs: on a
single-GPU box the test is skipped; its host-side shard arithmetic is covered on
CPU in test_tp_shards_cover_everything."""
import os
import socket

import numpy as np
import pytest

from oracle import gpt_oracle as O


def _shards(H, F, V, T):
    """Mirror of the shard arithmetic in rg_gpt_create (heads, hidden columns in 8s, vocabulary blocks)."""
    out = []
    vpad = -(-(-(-V // T)) // 8) * 8
    for r in range(T):
        hl, h0 = H // T + (1 if r < H % T else 0), r * (H // T) + min(r, H % T)
        f8 = F // 8
        fl, f0 = 8 * (f8 // T + (1 if r < f8 % T else 0)), 8 * (r * (f8 // T) + min(r, f8 % T))
        v0 = min(V, r * vpad)
        out.append((h0, hl, f0, fl, v0, max(0, min(vpad, V - v0))))
    return out


def test_tp_shards_cover_everything():
    for H, D, V, T in ((25, 1600, 50257, 8), (12, 768, 1024, 2), (3, 96, 301, 2), (16, 1024, 50257, 4)):
        sh = _shards(H, 4 * D, V, T)
        assert sum(s[1] for s in sh) == H and all(a[0] + a[1] == b[0] for a, b in zip(sh, sh[1:]))
        assert sum(s[3] for s in sh) == 4 * D and all(a[2] + a[3] == b[2] for a, b in zip(sh, sh[1:]))
        assert sum(s[5] for s in sh) == V and all(a[4] + a[5] == b[4] for a, b in zip(sh, sh[1:]))
        assert sh[0][1] - sh[-1][1] <= 1      # 25 heads over 8 ranks: 4,3,3,3,3,3,3,3


def _rank(rank, world, port, q, allreduce):
    os.environ["RG_B200_TP_ALLREDUCE"] = allreduce
    import torch
    import torch.distributed as dist
    import rustygradients_b200 as rg
    from helpers import F32_TOL, BF16_REL_TOL, teacher_forced
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)   # host channel for the 128-byte id only
    torch.cuda.set_device(rank)
    be = rg.B200Backend(rank)
    results = {}
    for name, cfg, dtype, B in (("f32", O.GptConfig(48, 301, 2, 3, 96), "f32", 2),
                                ("bf16", O.GptConfig(48, 1000, 2, 5, 320), "bf16", 3),
                                # 1 and 4 sequences, uneven heads (3 + 2): generate() runs as ONE persistent launch per rank
                                ("bf16_one", O.GptConfig(48, 1000, 3, 5, 320), "bf16", 1),
                                ("f32_four", O.GptConfig(48, 301, 2, 3, 96), "f32", 4),
                                # 9 sequences: the GEMM form of the token step with its row-split all-reduces
                                ("bf16_rows", O.GptConfig(48, 1000, 2, 5, 320), "bf16", 9)):
        params = O.make_params(cfg, 31, stress=True, bf16=(dtype == "bf16"))
        prompt = O.make_prompt(cfg, 31, B, 10)
        toks, want = O.generate_causal(params, cfg, prompt, 12)
        m = rg.GPTModel(be, rg.GptConfig(cfg.block_size, cfg.vocab_size, cfg.num_layers, cfg.num_heads, cfg.embedding_dim,
                                         weight_dtype=dtype, max_batch=max(4, B), tp_rank=rank, tp_size=world))
        m.load_parameters(params)
        ident = [rg.GPTModel.tp_unique_id() if rank == 0 else None]
        dist.broadcast_object_list(ident, src=0)
        m.tp_init(ident[0])
        fused = m.tp_fused()
        ids = np.concatenate([prompt, toks], 1)
        logits, picks = teacher_forced(m, ids, 10)
        err = np.abs(logits - want)
        rel = float((err / np.abs(want).max(-1, keepdims=True)).max())
        full = m.forward(ids[:, :20].astype(np.float32))
        ferr = float(np.abs(full - O.forward(params, cfg, ids[:, :20], causal=True, act="gelu_tanh")).max())
        l0 = be.launch_count
        out = m.generate(prompt, 12)
        gen_launches = be.launch_count - l0
        # ids against the oracle's wherever its top-2 gap is clear (up to the first unclear step of a sequence)
        tol = F32_TOL if dtype == "f32" else BF16_REL_TOL * float(np.abs(want).max())
        srt = np.sort(want, -1)
        sure = (srt[..., -1] - srt[..., -2]) > 4 * tol
        ids_ok = True
        for b in range(B):
            n = int(np.argmin(sure[b])) if not sure[b].all() else sure.shape[1]
            ids_ok &= bool(np.array_equal(out[b, :n], toks[b, :n]))
        results[name] = (float(err.max()), rel, ferr, bool(np.array_equal(picks, logits.argmax(-1))),
                         out.tolist(), F32_TOL, BF16_REL_TOL, fused, gen_launches, ids_ok)
        m.close()
    q.put((rank, results))
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.gpu
@pytest.mark.parametrize("allreduce", ["peer", "nccl"])
def test_tensor_parallel_two_gpus(allreduce):
    """allreduce = "peer": the token step's all-reduces are the library's one-shot kernel over peer-mapped memory
    (and must really be: tp_fused); "nccl": the same step with NCCL collectives."""
    import torch
    import torch.multiprocessing as mp
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_rank, args=(r, 2, port, q, allreduce)) for r in range(2)]
    [p.start() for p in procs]
    res = dict(q.get(timeout=600) for _ in range(2))
    [p.join(60) for p in procs]
    for name in ("f32", "bf16", "bf16_rows", "bf16_one", "f32_four"):
        a, b = res[0][name], res[1][name]
        assert a[4] == b[4]                                   # both ranks generate the same ids
        for maxabs, rel, ferr, picks_ok, _, f32_tol, bf16_tol, fused, gen_launches, ids_ok in (a, b):
            assert picks_ok and ids_ok
            assert fused == (allreduce == "peer")
            if allreduce == "peer" and name in ("f32", "bf16_one", "f32_four"):
                assert gen_launches < 150, gen_launches      # prompt pass + ONE launch for the 11 cached steps
            if name.startswith("f32"):
                assert maxabs <= f32_tol and ferr <= f32_tol
            else:
                assert rel <= bf16_tol
