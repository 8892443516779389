"""Tensor-parallel run on 2, 4 and 8 GPUs (NCCL, then the peer-memory exchange kernels: the all-reduce pushed
from the row-parallel GEMM's epilogue, and the pull variant) against the unsharded model on one GPU, same seed.
Each case is skipped when fewer GPUs are visible.  NVLink multicast stays off in every library used
(NCCL_NVLS_ENABLE=0; the symmetric buffer is never bound to a multicast object), the ranks meet at a host-side
barrier with idle GPUs before they leave, and every device-side wait is bounded."""

import os
import socket
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank: int, world: int, port: int, results):
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    os.environ["TORCH_SYMM_MEM_DISABLE_MULTICAST"] = "1"
    import torch.distributed as dist

    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    host = dist.new_group(backend="gloo")
    try:
        from xax_b200 import _lib
        from xax_b200.arch.llm import LLM, DecodeState, LLMConfig
        from xax_b200.parallel import TensorParallel

        cfg = LLMConfig(vocab_size=1024, embed_dim=512, q_heads=8, kv_heads=4 if world <= 4 else 8, head_dim=64,
                        num_layers=3, mlp_hidden_dim=1024, rms_eps=1e-5)
        B, T = 4, 48
        toks = torch.randint(0, 1024, (B, T), generator=torch.Generator().manual_seed(3), dtype=torch.int32).to(dev)
        tp = TensorParallel(rank, world)
        m = LLM.build(cfg, key=5, use_fp8=True, init_std=0.05, device=dev, tp_rank=rank, tp_size=world)
        tp.prepare_model(m)
        tp.shard_lm_head(m)
        st = DecodeState(m, B, T + 8, tp=tp)
        first = st.prefill(toks).clone()
        st.capture()
        seq = [first]
        for _ in range(3):
            seq.append(st.replay().clone())
        _lib.device_status()
        # one block, sharded vs unsharded, same input
        full = LLM.build(cfg, key=5, use_fp8=True, init_std=0.05, device=dev)
        x = (torch.randn((B * T, 512), generator=torch.Generator(device=dev).manual_seed(1), device=dev)).to(torch.bfloat16)
        y_tp, _ = tp.block_forward(m.blocks[0], x, B, T)
        y_1, _ = full.blocks[0].forward_tokens(x, B, T)
        err = float((y_tp.float() - y_1.float()).norm() / y_1.float().norm())
        # sharded e4m3 weights are slices of the unsharded ones
        q_full = full.blocks[0].self_attn.output_proj.weight_q_current()[0].view(torch.uint8)
        q_loc = m.blocks[0].self_attn.output_proj._wq_current[0].view(torch.uint8)
        n = q_full.shape[1] // world
        same_bytes = bool(torch.equal(q_loc, q_full[:, rank * n:(rank + 1) * n]))
        st1 = DecodeState(full, B, T + 8)
        first1 = st1.prefill(toks).clone()
        agree = float((first1 == first).float().mean())
        gathered = [torch.empty_like(first) for _ in range(world)]
        dist.all_gather(gathered, first)
        consistent = all(bool(torch.equal(g, first)) for g in gathered)
        # the same decode through the library's own peer-memory exchange kernels instead of NCCL
        tp2 = TensorParallel(rank, world)
        tp2.enable_peer_exchange(dev, rows=B, cols=512)
        vals = (torch.arange(B, device=dev, dtype=torch.float32) + 1) * (rank + 1)
        vmax = tp2.all_reduce_max(vals.clone())
        max_ok = bool(torch.equal(vmax, (torch.arange(B, device=dev, dtype=torch.float32) + 1) * world))
        sum_ok = True
        for it in range(5):  # alternates the two data buffers; compared with a gather + rank-ordered sum
            part = tp2.partial_out(B, 512)
            part.copy_(torch.randn((B, 512), generator=torch.Generator(device=dev).manual_seed(100 * it + rank),
                                   device=dev).to(torch.bfloat16))
            parts = [torch.empty_like(part) for _ in range(world)]
            dist.all_gather(parts, part.clone())
            want = torch.zeros((B, 512), dtype=torch.float32, device=dev)
            for q in parts:
                want += q.float()
            got = tp2.all_reduce_sum(part)
            sum_ok = sum_ok and bool(torch.equal(got, want.to(torch.bfloat16)))
        # the exchange fused with RMSNorm + per-token cast against exchange, then rmsnorm with a fused cast
        from xax_b200 import ops
        norm = m.blocks[0].mlp_norm
        fused_ok = True
        for it in range(2):
            src = torch.randn((B, 512), generator=torch.Generator(device=dev).manual_seed(500 + 10 * it + rank),
                              device=dev).to(torch.bfloat16)
            part = tp2.partial_out(B, 512)
            part.copy_(src)
            x_a = tp2.all_reduce_sum(part)
            _, (q_a, _, inv_a) = ops.rmsnorm(x_a, norm.weight_bf16(), norm.eps, want_y=False, quantize=True)
            part = tp2.partial_out(B, 512)
            part.copy_(src)
            x_b, q_b, inv_b = tp2.all_reduce_sum_norm(part, norm)
            fused_ok = fused_ok and bool(torch.equal(x_a, x_b) and torch.equal(inv_a, inv_b)
                                         and torch.equal(q_a.view(torch.uint8), q_b.view(torch.uint8)))
        # SiLU*up with the row-amax exchange inside the kernel against kernel, NCCL max, cast
        gu = torch.randn((B, 2 * 256), generator=torch.Generator(device=dev).manual_seed(900 + rank), device=dev
                         ).to(torch.bfloat16)
        hmax = torch.zeros((B,), dtype=torch.float32, device=dev)
        h, _ = ops.silu_mul(gu, 256, group_amax=hmax, group_rows=1)
        tp.all_reduce_max(hmax)
        hq_a, _, hinv_a = ops.quantize_with_amax(h, hmax, 1)
        for _ in range(3):  # repeated: the inbox copies alternate
            hq_b, _, hinv_b = ops.silu_mul_cast_tp(gu, 256, tp2.peer.silu_site())
            fused_ok = fused_ok and bool(torch.equal(hq_a.view(torch.uint8), hq_b.view(torch.uint8))
                                         and torch.equal(hinv_a, hinv_b))
        if tp2.peer.exchanges & 1:  # keep the buffer alternation even before capturing a graph
            tp2.all_reduce_sum(tp2.partial_out(B, 512).zero_())
        st2 = DecodeState(m, B, T + 8, tp=tp2)
        first2 = st2.prefill(toks).clone()
        st2.capture()
        seq2 = [first2]
        for _ in range(3):
            seq2.append(st2.replay().clone())
        _lib.device_status()
        peer_same = all(bool(torch.equal(a, b)) for a, b in zip(seq, seq2))
        # the same again with the pull variant of the sum (the GEMM writes locally, the sum kernel reads the
        # peers' rows): same arithmetic in the same order, so the tokens are the push run's
        tp4 = TensorParallel(rank, world, push=False)
        tp4.peer = tp2.peer
        st4 = DecodeState(m, B, T + 8, tp=tp4)
        seq4 = [st4.prefill(toks).clone()]
        st4.capture()
        for _ in range(3):
            seq4.append(st4.replay().clone())
        _lib.device_status()
        push_same = tp2.push and all(bool(torch.equal(a, b)) for a, b in zip(seq2, seq4))
        # per-rank-slice scaling (opt-in deviation): still the projection's output, to FP8 accuracy
        tp3 = TensorParallel(rank, world, local_amax=True)
        tp3.peer = tp2.peer
        y_loc, _ = tp3.block_forward(m.blocks[0], x, B, T)
        err_local = float((y_loc.float() - y_1.float()).norm() / y_1.float().norm())
        xd = x[:B].contiguous()
        cache_a = m.blocks[0].self_attn.init_cache(16, batch=B, device=dev)
        cache_b = m.blocks[0].self_attn.init_cache(16, batch=B, device=dev)
        if tp2.peer.exchanges & 1:
            tp2.all_reduce_sum(tp2.partial_out(B, 512).zero_())
        yd_g, _ = tp2.block_forward(m.blocks[0], xd, B, 1, cache=cache_a)
        yd_l, _ = tp3.block_forward(m.blocks[0], xd, B, 1, cache=cache_b)
        err_local_decode = float((yd_l.float() - yd_g.float()).norm() / yd_g.float().norm())
        results[rank] = dict(err=err, same_bytes=same_bytes, agree=agree, consistent=consistent, max_ok=max_ok,
                             push_same=push_same,
                             err_local=err_local, err_local_decode=err_local_decode,
                             sum_ok=sum_ok, peer_same=peer_same, fused_ok=fused_ok)
    except Exception:  # noqa: BLE001
        import traceback

        results[rank] = traceback.format_exc()
    finally:
        # A process group whose collectives were captured in a CUDA graph can block in
        # destroy_process_group; leave without tearing NCCL down (results are already stored).  The ranks
        # first drain their GPUs and meet on the host, so nobody leaves while a peer still waits on it.
        try:
            torch.cuda.synchronize()
            dist.barrier(group=host)
        except Exception:  # noqa: BLE001  (a rank that failed may never arrive: the others time out and leave)
            pass
        sys.stdout.flush()
        os._exit(0)


@pytest.mark.parametrize("world", [2, 4, 8])
def test_tensor_parallel_matches_one_gpu(world):
    import torch.multiprocessing as mp

    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    with mp.Manager() as mgr:
        results = mgr.dict()
        mp.spawn(_worker, args=(world, _free_port(), results), nprocs=world, join=True)
        res = dict(results)
    for r in range(world):
        assert isinstance(res[r], dict), res[r]
        msg = f"rank {r}: " + ", ".join(f"{k}={v}" for k, v in res[r].items())
        # Partial sums travel as bf16, so one block differs from the unsharded one by bf16 rounding -- of
        # `world` partial sums per row-parallel projection -- amplified by the two FP8 casts inside the block:
        # below 3e-2 at 2 and 4 ranks, 3.8e-2 measured at 8, where two executions of a block by the reference's
        # own two formulations (quantise-dequantise and FP8 matmul) differ by 4.4e-2.
        assert res[r]["err"] < (3e-2 if world <= 4 else 5e-2), msg
        assert res[r]["same_bytes"] and res[r]["consistent"], msg
        assert res[r]["agree"] >= 0.5, msg
        # peer-memory exchange: exact maximum, rank-ordered float32 sum, and (two ranks: one rounding of
        # a + b either way) the same greedy tokens as the NCCL run, prefill and three replayed steps
        # per-rank-slice scales put the e4m3 grid elsewhere than the unsharded model's: the block output moves
        # by FP8 rounding noise (the reference's own two executions of one block differ by 7e-2)
        assert res[r]["err_local"] < (6e-2 if world <= 4 else 8e-2) and res[r]["err_local_decode"] < 6e-2, msg
        assert res[r]["max_ok"] and res[r]["sum_ok"] and res[r]["fused_ok"] and res[r]["push_same"], msg
        if world == 2:  # two ranks: a + b rounds the same either way, so NCCL's sum gives the same tokens
            assert res[r]["peer_same"], msg
