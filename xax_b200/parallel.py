"""Tensor parallelism over the GPUs of one NVSwitch box, one process per GPU.

Placement follows xax/arch/llm.py:931-975 (``get_model_parallel_sharding_spec``): q/k/v/gate/up
and lm_head are split along ``out`` (column parallel), o_proj/down_proj along ``in`` (row
parallel); embeddings, norms and 1-D tensors are replicated.  The reference leaves the
collectives to XLA/GSPMD (an all-reduce after every row-parallel matmul); here they are explicit:

  * the partial outputs of o_proj and down_proj are summed across ranks (``all_reduce_sum``);
  * the activation feeding a row-parallel FP8 layer is sharded along the reduction dimension,
    so its amax (per token for o_proj, per sequence for down_proj) is max-reduced across ranks
    before the cast -- the e4m3 bytes then equal the unsharded model's;
  * greedy decoding needs no logits gather: each rank arg-maxes its vocabulary slice and the
    (value, index) pairs are all-gathered and merged.

Collectives go through ``torch.distributed`` (NCCL over NVLink on GPUs, gloo in CPU tests).  On
GPUs the two exchanges of the decode step can instead run as this library's own kernels over
peer memory (``TensorParallel.enable_peer_exchange``): the row-parallel GEMM writes its partial
output into a buffer that every GPU of the box has mapped, and one kernel per exchange waits on
flags in that buffer and reads the peers' rows directly over NVLink.
"""

from __future__ import annotations

import torch
import torch.distributed as dist

from .arch.llm import get_model_parallel_sharding_spec, tp_shard_dim  # noqa: F401  (re-exported)


def setup_model_parallel_mesh(mp_size: int | None = None) -> dict:
    """xax/arch/llm.py:907-928 for one-process-per-GPU launches: returns {"axis": "model",
    "size", "rank"} from the initialised process group (``mp_size`` must equal its size)."""
    if not dist.is_initialized():
        if mp_size not in (None, 1):
            raise ValueError(f"mp_size ({mp_size}) > available devices (1): launch one process per GPU with torchrun")
        return {"axis": "model", "size": 1, "rank": 0}
    world = dist.get_world_size()
    if mp_size is not None and mp_size > world:
        raise ValueError(f"mp_size ({mp_size}) > available devices ({world})")
    if mp_size is not None and mp_size != world:
        raise ValueError("a tensor-parallel group smaller than the launch is not supported")
    return {"axis": "model", "size": world, "rank": dist.get_rank()}


def shard_weight(weight: torch.Tensor, weight_name: str, rank: int, size: int) -> torch.Tensor:
    """This rank's slice of a weight under the placement rule (replicated weights are returned whole)."""
    dim = tp_shard_dim(weight_name, weight.dim())
    if size == 1 or dim is None:
        return weight
    if weight.shape[dim] % size:
        raise ValueError(f"{weight_name}: dimension {dim} of {tuple(weight.shape)} does not divide by {size}")
    n = weight.shape[dim] // size
    return weight.narrow(dim, rank * n, n).contiguous()


def make_sharded_array(arr: torch.Tensor, weight_name: str, rank: int, size: int, device=None) -> torch.Tensor:
    """What the checkpoint loader's ``make_sharded_array`` (xax/arch/llm.py:1244-1265) hands one
    device: this rank's slice of ``arr`` under the placement rule, or all of it when the rule
    replicates the tensor."""
    out = shard_weight(arr, weight_name, rank, size) if size > 1 else arr
    return out.to(device) if device is not None else out


class PeerExchange:
    """One symmetric buffer per rank, mapped by every rank of the box, laid out as
    [flag regions | amax inboxes | arg-max inbox and flags | data 0 | data 1], and the kernels that exchange through
    it.  The buffer and its mappings come from ``torch.distributed._symmetric_memory`` (plumbing);
    flags, protocol and kernels are this library's (``csrc/tp_collectives.cu``)."""

    MAX_ROWS = 1024

    def __init__(self, rank: int, size: int, group, device, rows: int, cols: int):
        import ctypes
        import os

        # The kernels use plain peer loads and stores only.  Left alone, torch would also bind the
        # buffer to an NVLink multicast object on an NVSwitch box; nothing here needs it, and a rank
        # that exits while its memory is bound to one can fault the other ranks' GPUs.
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
        import torch.distributed._symmetric_memory as symm

        from . import _lib

        lib = _lib.load()
        if not 1 <= rows <= self.MAX_ROWS or cols % 8:
            raise ValueError(f"peer exchange covers up to {self.MAX_ROWS} rows and a multiple of 8 columns")
        self.rank, self.size, self.rows, self.cols = rank, size, rows, cols

        def up(n):
            return (n + 4095) // 4096 * 4096

        sync = up(lib.xaxb_tp_sync_bytes())
        box = up(lib.xaxb_tp_max_inbox_bytes())
        # flag regions: sum, vector max, per-row max inside SiLU*up, per-row max inside attention
        self.sum_sync, self.max_sync, self.silu_sync, self.attn_sync = 0, sync, 2 * sync, 3 * sync
        self.inbox = 4 * sync
        self.silu_inbox, self.attn_inbox = self.inbox + box, self.inbox + 2 * box
        self.argmax_inbox = self.inbox + 3 * box
        self.argmax_sync = self.argmax_inbox + up(lib.xaxb_tp_argmax_inbox_bytes())
        self.data = [self.argmax_sync + sync]
        self.data.append(self.data[0] + up(rows * cols * 2))
        # push exchange: two (arrival counter, staging buffer of `size` slots) pairs used in alternation
        self.slot = up(rows * cols * 2)
        self.push_flag = [self.data[1] + up(rows * cols * 2), self.data[1] + up(rows * cols * 2) + 4096]
        self.push_data = [self.push_flag[1] + 4096, self.push_flag[1] + 4096 + size * self.slot]
        total = self.push_data[1] + size * self.slot
        self.buf = symm.empty(total, dtype=torch.uint8, device=device)
        self.buf.zero_()
        self.handle = symm.rendezvous(self.buf, group if group is not None else dist.group.WORLD)
        ptrs = list(self.handle.buffer_ptrs)
        if len(ptrs) != size or ptrs[rank] != self.buf.data_ptr():
            raise RuntimeError("symmetric-memory rendezvous returned an unexpected mapping table")
        self.peer_ptrs = (ctypes.c_void_p * size)(*ptrs)
        torch.cuda.synchronize(device)
        dist.barrier(group)  # every rank's flags are zero before anyone raises one
        self.exchanges = 0  # sum exchanges issued (or captured) so far: picks the data buffer
        self.pushes = 0     # push exchanges issued (or captured) so far: picks the (counter, staging) pair
        self.push_totals = torch.zeros((2, lib.xaxb_tp_push_totals_bytes() // 4), dtype=torch.int32, device=device)

    def partial_out(self, rows: int, cols: int) -> torch.Tensor:
        """Where the next row-parallel GEMM must write its partial output (bf16 [rows, cols])."""
        if rows > self.rows or cols != self.cols:
            raise ValueError(f"peer exchange was sized for [{self.rows}, {self.cols}], got [{rows}, {cols}]")
        off = self.data[self.exchanges & 1]
        return self.buf[off:off + rows * cols * 2].view(torch.bfloat16).view(rows, cols)

    def all_reduce_sum(self, partial: torch.Tensor) -> torch.Tensor:
        from . import ops

        off = self.data[self.exchanges & 1]
        if partial.data_ptr() != self.buf.data_ptr() + off:
            raise ValueError("the partial output must be the tensor partial_out() returned for this exchange")
        rows, cols = partial.shape
        out = torch.empty((rows, cols), dtype=torch.bfloat16, device=partial.device)
        ops.tp_allreduce_sum(self.peer_ptrs, self.rank, self.size, off, self.sum_sync, rows, cols, out)
        self.exchanges += 1
        return out

    def all_reduce_sum_norm(self, partial: torch.Tensor, weight_bf16: torch.Tensor, eps: float):
        """all_reduce_sum fused with RMSNorm and the per-token e4m3 cast of the summed rows:
        (x bf16, q e4m3, inv_scale float32 [rows])."""
        from . import ops

        off = self.data[self.exchanges & 1]
        if partial.data_ptr() != self.buf.data_ptr() + off:
            raise ValueError("the partial output must be the tensor partial_out() returned for this exchange")
        rows, cols = partial.shape
        x, q, _, inv = ops.tp_allreduce_sum_rmsnorm(self.peer_ptrs, self.rank, self.size, off, self.sum_sync, rows, cols,
                                                    weight_bf16, eps)
        self.exchanges += 1
        return x, q, inv

    def push_target(self, rows: int, cols: int) -> "PushTarget":
        """Where the next row-parallel GEMM of a decode step pushes its partial output."""
        if rows > self.rows or cols != self.cols or rows > 128:
            raise ValueError(f"push exchange covers up to {min(self.rows, 128)} rows of {self.cols} columns")
        return PushTarget(self, self.pushes & 1, rows, cols)

    def silu_site(self):
        """Arguments that route the SiLU*up kernel's row-amax exchange through this buffer."""
        return (self.peer_ptrs, self.rank, self.size, self.silu_inbox, self.silu_sync)

    def attn_site(self):
        return (self.peer_ptrs, self.rank, self.size, self.attn_inbox, self.attn_sync)

    def all_reduce_max(self, values: torch.Tensor) -> torch.Tensor:
        from . import ops

        return ops.tp_allreduce_max(self.peer_ptrs, self.rank, self.size, self.inbox, self.max_sync, values)


class PushTarget:
    """One push exchange: the row-parallel GEMM writes its partial output into this rank's slot of every
    rank's staging buffer from its epilogue (``push_gemm``); ``sum_norm`` then waits for every rank's pieces
    and reduces them from local memory.  Made by PeerExchange.push_target; used once."""

    def __init__(self, peer: PeerExchange, parity: int, rows: int, cols: int):
        self.peer, self.parity, self.rows, self.cols = peer, parity, rows, cols
        self.pushed = False

    def push_gemm(self, xq, wq, x_inv, w_inv, bias, residual) -> "PushTarget":
        from . import ops

        p = self.peer
        if xq.shape[0] != self.rows or wq.shape[0] != self.cols:
            raise ValueError(f"push target was made for [{self.rows}, {self.cols}], got [{xq.shape[0]}, {wq.shape[0]}]")
        ops.gemm_fp8_push(xq, wq, x_inv, w_inv, bias, residual, p.peer_ptrs, p.rank, p.size,
                          p.push_data[self.parity] + p.rank * p.slot, p.push_flag[self.parity])
        self.pushed = True
        p.pushes += 1
        return self

    def sum_norm(self, weight_bf16=None, eps: float = 0.0):
        """(x, q, inv_scale) with a norm weight, (x, None, None) without."""
        from . import ops

        if not self.pushed:
            raise ValueError("nothing was pushed to this target")
        p = self.peer
        base = p.buf.data_ptr()
        x, q, _, inv = ops.tp_push_sum_rmsnorm(base + p.push_data[self.parity], p.slot, base + p.push_flag[self.parity],
                                               p.push_totals[self.parity].data_ptr(), p.size, self.rows, self.cols,
                                               p.buf.device, weight_bf16, eps)
        return x, q, inv


class TensorParallel:
    """Collectives and the tensor-parallel forward of one transformer block."""

    def __init__(self, rank: int, size: int, group=None, local_amax: bool = False, push: bool = True):
        """``local_amax=False`` (default) keeps the reference's numerics: the activations feeding the
        row-parallel FP8 layers are cast with the amax of the WHOLE row, max-reduced over the ranks, so
        their e4m3 bytes equal the unsharded model's.  ``local_amax=True`` casts each rank's slice with
        the slice's own amax (the partial products are dequantised per rank, so the sum is still the
        projection's output, at a finer scaling granularity than the reference's): two of the four
        exchanges per block disappear.  It is a deviation from the reference and is never the default."""
        self.rank, self.size, self.group = rank, size, group
        self.local_amax = bool(local_amax)
        # decode steps: the row-parallel GEMMs push their partial outputs to every rank from the epilogue
        # (False: they write locally and the sum kernel pulls the rows from the peers)
        self.push = bool(push)
        self.peer: PeerExchange | None = None
        if size > 1 and torch.cuda.is_available():
            # Programmatic dependent launch (successors scheduled early, waiting on the device) next
            # to kernels that wait for other GPUs, measured on 8 layers of the cfg5 decode step:
            # two GPUs 1.63 ms with it against 1.69 ms without, four GPUs 1.33 ms against 1.27 ms.
            # It stays as the process has it (on by default) for two ranks and is switched off beyond.
            if size > 2:
                from . import _lib

                _lib.load().xaxb_set_programmatic_launch(0)

    def enable_peer_exchange(self, device, rows: int, cols: int) -> None:
        """Route the decode step's exchanges ([<= rows, cols] partial outputs, <= rows amax values)
        through peer memory instead of NCCL.  Larger shapes (prefill) keep using NCCL.  A captured
        CUDA graph must hold an even number of sum exchanges (two per block: it does), so that the
        two data buffers keep alternating from one replay to the next."""
        if self.size <= 1:
            return
        # Every rank must end up on the same path: if setting up the shared buffer fails anywhere
        # (no peer access, symmetric memory unavailable), all ranks stay on NCCL.
        peer, err = None, None
        try:
            peer = PeerExchange(self.rank, self.size, self.group, device, rows, cols)
        except Exception as e:  # noqa: BLE001
            err = e
        ok = torch.tensor([0 if peer is None else 1], dtype=torch.int32, device=device)
        dist.all_reduce(ok, op=dist.ReduceOp.MIN, group=self.group)
        if int(ok.item()) == 1:
            self.peer = peer
        elif self.rank == 0:
            import warnings

            warnings.warn(f"peer-memory exchange unavailable ({err!r}); tensor-parallel exchanges stay on NCCL")

    def _peer_fits(self, rows: int, cols: int) -> bool:
        return self.peer is not None and rows <= self.peer.rows and cols == self.peer.cols

    # -- collectives ------------------------------------------------------------------------------
    def partial_out(self, rows: int, cols: int, decode: bool = False):
        """Output of a row-parallel GEMM whose result all_reduce_sum(_norm) will take next: a push target for
        a decode step on the push path, else the tensor in the symmetric buffer the peers pull from, else
        None (let the GEMM allocate; the exchange then goes through NCCL)."""
        if not self._peer_fits(rows, cols):
            return None
        if decode and self.push and rows <= 128:
            return self.peer.push_target(rows, cols)
        return self.peer.partial_out(rows, cols)

    def all_reduce_sum(self, t) -> torch.Tensor:
        if isinstance(t, PushTarget):
            return t.sum_norm()[0]
        if self.size > 1:
            if self.peer is not None and t.dim() == 2 and self._peer_fits(*t.shape) and \
                    t.data_ptr() == self.peer.partial_out(*t.shape).data_ptr():
                return self.peer.all_reduce_sum(t)
            dist.all_reduce(t, op=dist.ReduceOp.SUM, group=self.group)
        return t

    def all_reduce_sum_norm(self, t: torch.Tensor, norm):
        """Sum of the partial outputs, then ``norm`` (an RMSNorm) and the per-token e4m3 cast of the
        result: (x, q, inv_scale).  One kernel on the peer-memory path."""
        from . import ops

        w = norm.weight_bf16()
        if isinstance(t, PushTarget):
            return t.sum_norm(w, norm.eps)
        if self.size > 1 and self.peer is not None and t.dim() == 2 and self._peer_fits(*t.shape) and \
                t.shape[1] <= 8192 and t.data_ptr() == self.peer.partial_out(*t.shape).data_ptr():
            return self.peer.all_reduce_sum_norm(t, w, norm.eps)
        x = self.all_reduce_sum(t)
        _, yq = ops.rmsnorm(x, w, norm.eps, want_y=False, quantize=True)
        return x, yq[0], yq[2]

    def all_reduce_max(self, t: torch.Tensor) -> torch.Tensor:
        if self.size > 1:
            if self.peer is not None and t.is_cuda and t.dtype == torch.float32 and t.dim() == 1 and \
                    t.numel() <= PeerExchange.MAX_ROWS and t.is_contiguous():
                return self.peer.all_reduce_max(t)
            dist.all_reduce(t, op=dist.ReduceOp.MAX, group=self.group)
        return t

    def all_gather(self, t: torch.Tensor) -> torch.Tensor:
        out = torch.empty((self.size, *t.shape), dtype=t.dtype, device=t.device)
        if self.size == 1:
            out[0] = t
        elif t.is_cuda:
            dist.all_gather_into_tensor(out, t.contiguous(), group=self.group)
        else:  # gloo
            parts = [torch.empty_like(t) for _ in range(self.size)]
            dist.all_gather(parts, t.contiguous(), group=self.group)
            out = torch.stack(parts)
        return out

    # -- model pieces -----------------------------------------------------------------------------
    def prepare_model(self, model) -> None:
        """Quantise every sharded FP8 weight with the amax of the WHOLE weight (max over ranks),
        so each rank's e4m3 bytes are the corresponding slice of the unsharded model's."""
        from . import ops
        from .nn.fp8 import Fp8Linear

        for block in model.blocks:
            a, f = block.self_attn, block.feed_forward
            for lin in (a.q_proj, a.k_proj, a.v_proj, a.output_proj, f.gate, f.up, f.down):
                if isinstance(lin, Fp8Linear) and lin.use_fp8:
                    w = lin.weight.to(torch.bfloat16).contiguous()
                    amax = ops.group_amax(w, w.shape[0])
                    self.all_reduce_max(amax)
                    q, _, inv = ops.quantize_with_amax(w, amax, w.shape[0])
                    lin.set_weight_q_current(q, inv[:1].clone())
            a._fused = None
            f._fused = None

    def shard_lm_head(self, model) -> None:
        """Keep only this rank's vocabulary slice of the lm_head (column parallel, :970-972)."""
        from .arch.attention import Linear

        w = model.lm_head.weight
        if w.shape[0] % self.size:
            raise ValueError(f"vocabulary {w.shape[0]} does not divide by {self.size}")
        n = w.shape[0] // self.size
        model.lm_head = Linear(w.shape[1], n, use_bias=False, weight=w.narrow(0, self.rank * n, n).contiguous())
        model.vocab_slice = n

    def greedy_tokens(self, model, hidden_bh: torch.Tensor, out: torch.Tensor) -> None:
        """argmax over the full vocabulary from per-rank slices, written to ``out`` int32 [B]."""
        from . import ops

        logits = ops.gemm_bf16(hidden_bh.contiguous(), model.lm_head.weight)
        B = logits.shape[0]
        idx = torch.empty((B,), dtype=torch.int32, device=logits.device)
        val = torch.empty((B,), dtype=torch.float32, device=logits.device)
        ops.argmax(logits, out=idx, max_out=val)
        if self.peer is not None and B <= PeerExchange.MAX_ROWS:
            p = self.peer
            ops.tp_argmax(p.peer_ptrs, p.rank, p.size, p.argmax_inbox, p.argmax_sync, val, idx, logits.shape[1], out)
        else:
            ops.argmax_merge(self.all_gather(val), self.all_gather(idx), logits.shape[1], out)

    def block_forward(self, block, x: torch.Tensor, B: int, T: int, *, cache=None, workspace=None,
                      advance: bool = True):
        """One pre-norm block with this rank's weight shards.  x [B*T, H] is replicated on entry
        and on exit.  The residual is added by rank 0's GEMM epilogue only, so the sum of the
        partial outputs is x + f(x)."""
        x2, new_cache, _ = self.block_forward_chain(block, x, B, T, cache=cache, workspace=workspace, advance=advance)
        return x2, new_cache

    def block_forward_chain(self, block, x: torch.Tensor, B: int, T: int, *, cache=None, workspace=None,
                            advance: bool = True, x_q=None, next_norm=None):
        """block_forward for a chain of blocks in a decode step: ``x_q`` = (q, inv_scale), the
        attn_norm + cast of x if the previous block's closing exchange already produced it;
        ``next_norm`` = the norm that will consume this block's output (the next block's attn_norm),
        to be fused into this block's closing exchange.  Returns (x, cache, next x_q or None)."""
        from . import ops

        attn, ff = block.self_attn, block.feed_forward
        first = self.rank == 0
        if not (attn._is_fp8() and ff.is_fp8()):
            raise ValueError("the tensor-parallel path covers FP8 projections (use_fp8=True)")
        if x_q is None:
            _, yq = ops.rmsnorm(x, block.attn_norm.weight_bf16(), block.attn_norm.eps, want_y=False, quantize=True)
            x_q = (yq[0], yq[2])
        local = self.local_amax
        fused = T == 1 and not local and self._peer_fits(B, x.shape[1])  # amax exchanges inside the producers
        part, new_cache = attn.forward_tokens(x, B, T, cache=cache, y_q=x_q, residual=x if first else None,
                                              workspace=workspace, advance=advance,
                                              reduce_amax=None if local else self.all_reduce_max,
                                              out=self.partial_out(B * T, x.shape[1], decode=T == 1),
                                              peer_site=self.peer.attn_site() if fused else None)
        wq, col, bias = ff.fused_gate_up()
        F = ff.gate.out_features  # local width
        if T == 1:
            x1, q, inv = self.all_reduce_sum_norm(part, block.mlp_norm)
        else:
            x1 = self.all_reduce_sum(part)
            amax = torch.zeros((B,), dtype=torch.float32, device=x.device)
            y, _ = ops.rmsnorm(x1, block.mlp_norm.weight_bf16(), block.mlp_norm.eps, group_amax=amax, group_rows=T)
            q, _, inv = ops.quantize_with_amax(y, amax, T)
        gu = ops.gemm_fp8(q, wq, inv, col, bias)
        if fused:
            hq, _, h_inv = ops.silu_mul_cast_tp(gu, F, self.peer.silu_site())
        elif local and T == 1:
            _, (hq, _, h_inv) = ops.silu_mul(gu, F, want_h=False, quantize=True)
        elif local:
            hmax = torch.zeros((B,), dtype=torch.float32, device=x.device)
            h, _ = ops.silu_mul(gu, F, group_amax=hmax, group_rows=T)
            hq, _, h_inv = ops.quantize_with_amax(h, hmax, T)
        else:
            hmax = torch.zeros((B,), dtype=torch.float32, device=x.device)
            h, _ = ops.silu_mul(gu, F, group_amax=hmax, group_rows=T)
            self.all_reduce_max(hmax)  # the down projection's input spans all ranks
            hq, _, h_inv = ops.quantize_with_amax(h, hmax, T)
        part = ff.down.forward_quantized(hq, h_inv, x1 if first else None,
                                         self.partial_out(B * T, x.shape[1], decode=T == 1))
        if next_norm is not None and T == 1:
            x2, q2, inv2 = self.all_reduce_sum_norm(part, next_norm)
            return x2, new_cache, (q2, inv2)
        return self.all_reduce_sum(part), new_cache, None
