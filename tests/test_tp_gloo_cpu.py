"""Tensor-parallel host logic on two gloo ranks (CPU): the placement rule, and the algorithm the
GPU path runs -- amax max-reduced across ranks before the cast so e4m3 bytes equal the unsharded
model's, partial outputs of a row-parallel layer sum-reduced, column-parallel outputs
concatenated, vocabulary-sharded arg-max merged -- executed with the oracle's arithmetic."""

import os
import socket
import sys

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank: int, world: int, port: int, results):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, HERE)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from helpers import bf16, cfg1_inputs, e4m3, f32
        from oracle import fp8 as ofp8
        from xax_b200.parallel import TensorParallel, setup_model_parallel_mesh, shard_weight

        mesh = setup_model_parallel_mesh(world)
        assert mesh == {"axis": "model", "size": world, "rank": rank}
        tp = TensorParallel(rank, world)
        x, w, b, rng = cfg1_inputs(M=16, K=256, N=64, seed=7)  # identical on every rank
        wt = torch.from_numpy(f32(w))

        # ---- row parallel (o_proj / down_proj): shard `in`, amax of activation and weight max-reduced
        w_row = shard_weight(wt, "layers.0.self_attn.o_proj", rank, world).numpy().astype(bf16)
        k0 = rank * (256 // world)
        x_loc = x[:, k0:k0 + 256 // world]
        assert w_row.shape == (64, 256 // world)
        amax = torch.from_numpy(np.max(np.abs(f32(x_loc)), axis=1))
        tp.all_reduce_max(amax)
        assert np.array_equal(amax.numpy(), np.max(np.abs(f32(x)), axis=1))
        wamax = torch.tensor([float(np.max(np.abs(f32(w_row))))])
        tp.all_reduce_max(wamax)
        floor = f32(np.asarray(1e-12).astype(bf16))
        sx = (np.float32(448) / np.maximum(amax.numpy(), floor)).astype(bf16)
        sw = (np.float32(448) / np.maximum(wamax.numpy(), floor)).astype(bf16)[0]
        q_loc = ofp8.quantize(x_loc, e4m3, sx[:, None], bf16)
        qw_loc = ofp8.quantize(w_row, e4m3, sw, bf16)
        # bytes equal the corresponding slices of the unsharded cast
        layer = ofp8.Fp8Linear(w, None)
        _, sx_full, q_full = layer.call_rows(x)
        assert np.array_equal(sx.view(np.uint16), sx_full.view(np.uint16))
        assert np.array_equal(q_loc.view(np.uint8), q_full[:, k0:k0 + 256 // world].view(np.uint8))
        sw_full = ofp8.current_scale(w, e4m3, bf16)
        assert sw.view(np.uint16) == sw_full.view(np.uint16)
        part = (f32(q_loc) @ f32(qw_loc).T) * (1.0 / f32(sx))[:, None] * (1.0 / f32(sw))
        total = torch.from_numpy(part.astype(np.float32))
        tp.all_reduce_sum(total)
        ofp8.MATMUL_MODE = "fp8_gemm"
        exp = f32(layer.call_rows(x)[0])
        ofp8.MATMUL_MODE = "qdq"
        assert np.allclose(f32(total.numpy().astype(bf16)), exp, rtol=2e-2, atol=1e-3)

        # ---- column parallel (q/k/v/gate/up): shard `out`, results concatenate
        w_col = shard_weight(wt, "mlp.gate_proj", rank, world)
        assert w_col.shape == (64 // world, 256)
        out_loc = torch.from_numpy(f32(x) @ w_col.numpy().T)
        gathered = tp.all_gather(out_loc)  # [world, M, N/world]
        full = torch.cat(list(gathered), dim=1).numpy()
        assert np.allclose(full, f32(x) @ f32(w).T, rtol=1e-5, atol=1e-5)
        assert shard_weight(wt, "norm.weight", rank, world) is wt  # replicated

        # ---- vocabulary-sharded greedy token: local (max, index) pairs, gathered, lowest index on ties
        V, B = 32, 5
        logits = rng.standard_normal((B, V)).astype(np.float32)
        logits[1, 3] = logits[1, 20] = 9.0  # a tie across the two slices
        sl = logits[:, rank * (V // world):(rank + 1) * (V // world)]
        vals = tp.all_gather(torch.from_numpy(sl.max(axis=1)))
        idxs = tp.all_gather(torch.from_numpy(sl.argmax(axis=1).astype(np.int32)))
        best = np.full(B, -np.inf, np.float32)
        tok = np.zeros(B, np.int64)
        for p in range(world):
            v, i = vals[p].numpy(), idxs[p].numpy() + p * (V // world)
            take = v > best
            best, tok = np.where(take, v, best), np.where(take, i, tok)
        assert np.array_equal(tok, logits.argmax(axis=1))

        # ---- the push exchange's arithmetic: every rank holds every rank's bf16 partial output (its slot of
        # the staging buffer), sums the slots in rank order in float32 and rounds once -- so all ranks get the
        # same bits, whatever order the pieces arrived in
        part_bf = torch.from_numpy(part.astype(np.float32)).to(torch.bfloat16)
        slots = tp.all_gather(part_bf.view(torch.int16).to(torch.int32)).to(torch.int16).view(torch.bfloat16)  # [world, M, N]
        acc = torch.zeros(part_bf.shape, dtype=torch.float32)
        for r in range(world):
            acc += slots[r].float()
        mine = acc.to(torch.bfloat16)
        others = tp.all_gather(mine.view(torch.int16).to(torch.int32))
        assert all(torch.equal(others[r], mine.view(torch.int16).to(torch.int32)) for r in range(world))
        pieces = world * part_bf.shape[0] * part_bf.shape[1] // 8  # what each rank's arrival counter must reach
        assert pieces == world * 16 * 64 // 8

        # ---- make_sharded_array (xax/arch/llm.py:1244-1265): this rank's slice, or the whole tensor
        from xax_b200.parallel import make_sharded_array

        assert torch.equal(make_sharded_array(wt, "layers.3.mlp.down_proj", rank, world), wt[:, k0:k0 + 256 // world])
        assert torch.equal(make_sharded_array(wt, "layers.3.self_attn.q_proj", rank, world),
                           wt[rank * (64 // world):(rank + 1) * (64 // world)])
        assert make_sharded_array(wt, "layers.3.input_layernorm.weight", rank, world) is wt
        assert make_sharded_array(wt[0], "layers.3.mlp.up_proj.bias", rank, world).shape == (256,)  # 1-D: replicated
        results[rank] = "ok"
    except Exception as e:  # noqa: BLE001
        import traceback

        results[rank] = traceback.format_exc()
    finally:
        dist.destroy_process_group()


def test_tensor_parallel_algorithm_two_gloo_ranks():
    world = 2
    port = _free_port()
    with mp.Manager() as mgr:
        results = mgr.dict()
        mp.spawn(_worker, args=(world, port, results), nprocs=world, join=True)
        assert dict(results) == {0: "ok", 1: "ok"}, dict(results)


def test_mesh_without_process_group():
    from xax_b200.parallel import setup_model_parallel_mesh

    assert setup_model_parallel_mesh() == {"axis": "model", "size": 1, "rank": 0}
    try:
        setup_model_parallel_mesh(4)
    except ValueError as e:
        assert "available devices" in str(e)
    else:
        raise AssertionError("mp_size beyond the launch must raise like the reference")
