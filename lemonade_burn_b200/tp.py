"""Tensor-parallel sharding of packed ternary projections (one process per GPU, torch.distributed).

The reference has no multi-device path; the closest thing is its two-socket row split
(crates/lb-model/src/ops.rs:255-297, crates/lb-ternary/src/numa.rs:122-124), which this
generalises:

* column-parallel (q/k/v, gate, up): each rank holds a contiguous range of the packed ROWS -- no
  repacking, rows are contiguous in the lb-ternary layout (pack.rs:46-49). The input is
  replicated, every rank quantises the whole token row itself (identical on all ranks), outputs
  are sharded along features. No collective.
* row-parallel (o, down): each rank holds a range of the COLUMNS, a multiple of 128 so that the
  cut falls on packed-block boundaries (a contiguous byte range of every row, copied once at
  load). Per-token quantisation needs the maximum over the whole row, so ranks all-reduce (MAX)
  their slice maxima first; then every rank has the same scale, quantises its slice, computes
  exact int32 partial dots, and the partial dots are all-reduced with an integer SUM, which is
  exact and order independent. The scale epilogue runs after the reduction. Results are
  bit-identical to the single-GPU op for any world size.
"""
from __future__ import annotations

import ctypes as C
from typing import List, Optional, Sequence

import numpy as np

from .pack import BLOCK, row_bytes


# ---- pure host-side slicing (numpy or torch tensors; no GPU needed) -----------------------

def shard_rows(packed, world: int, rank: int):
    """Rows [rank*rows/world, (rank+1)*rows/world) of a packed [rows, row_bytes] matrix."""
    rows = packed.shape[0]
    if rows % world:
        raise ValueError(f"{rows} rows do not divide over {world} ranks")
    n = rows // world
    return packed[rank * n:(rank + 1) * n]


def shard_cols(packed, cols: int, world: int, rank: int):
    """Columns [rank*cols/world, (rank+1)*cols/world) of a packed matrix as a packed matrix of
    cols/world columns: a byte range of every row. Returns (slice view, local cols)."""
    if cols % world or (cols // world) % BLOCK:
        raise ValueError(f"{cols} columns over {world} ranks do not fall on 128-column blocks")
    if packed.shape[1] != row_bytes(cols):
        raise ValueError("packed data length mismatch")
    lc = cols // world
    lb = lc // 4
    return packed[:, rank * lb:(rank + 1) * lb], lc


# ---- peer-memory communicator for the fused row-parallel kernels --------------------------------

class TpComm:
    """One region of device memory per rank, opened in every rank through CUDA IPC handles that
    travel over the torch.distributed group (any transport would do), for lbk_tp_quantize /
    lbk_tp_reduce_scale. Plain NVLink peer loads and stores; NCCL is not involved in the data path."""

    def __init__(self, ctx, world: int, rank: int, group=None):
        import torch.distributed as dist
        from . import _lib
        self.ctx, self.world, self.rank = ctx, world, rank
        lib = ctx._lib
        self._lib = lib
        self.max_tokens = int(lib.lbk_tp_max_tokens())
        self.partial_bytes = int(lib.lbk_tp_partial_bytes())
        mine = C.c_void_p()
        handle = (C.c_ubyte * 64)()
        _lib.check(lib.lbk_tp_region_alloc(ctx.handle, C.byref(mine), handle))
        self._mine = mine
        handles = [None] * world
        if world > 1:
            dist.all_gather_object(handles, bytes(handle), group=group)
        else:
            handles[0] = bytes(handle)
        self._opened = []
        regions = []
        for r in range(world):
            if r == rank:
                regions.append(mine.value)
                continue
            ptr = C.c_void_p()
            buf = (C.c_ubyte * 64).from_buffer_copy(handles[r])
            _lib.check(lib.lbk_tp_region_open(ctx.handle, buf, C.byref(ptr)))
            self._opened.append(ptr)
            regions.append(ptr.value)
        arr, self._keep = _lib.ptr_array(regions)
        h = C.c_void_p()
        _lib.check(lib.lbk_tp_comm_create(ctx.handle, world, rank, arr, C.byref(h)))
        self.handle = h
        self.partial_ptr = int(lib.lbk_tp_partial_buffer(h))
        if world > 1:
            dist.barrier(group=group)  # every rank has opened every region before anyone launches

    def close(self):
        """Call on every rank once no kernel of the group is in flight."""
        if getattr(self, "handle", None):
            self._lib.lbk_tp_comm_destroy(self.handle)
            self.handle = None
            for ptr in self._opened:
                self._lib.lbk_tp_region_close(self.ctx.handle, ptr)
            self._lib.lbk_tp_region_free(self.ctx.handle, self._mine)


class PeerLost(RuntimeError):
    """A rank of the tensor-parallel group did not show up for a step."""


class PeerGuard:
    """Host-side liveness check between steps. The peer-memory kernels bound their waits and report
    LBK_ERR_TIMEOUT when a peer never arrives, but by then a step's worth of launches is queued; this
    check finds a missing rank BEFORE the next launch: every rank posts a key for the step in a
    key-value store (torch.distributed's TCPStore or any object with set / wait) and waits, with a
    timeout, for the keys of all ranks. A rank that left (or the store's host that went away) turns into
    PeerLost on the others, the same rule as the reference's server, where a failing request becomes an
    error reply and never a dead worker (crates/lb-server/src/main.rs:92-100). A rank leaves only
    between steps, with none of its kernels in flight."""

    def __init__(self, store, world: int, rank: int, timeout_s: float = 5.0, prefix: str = "lbk/alive"):
        self.store, self.world, self.rank, self.timeout_s, self.prefix = store, world, rank, timeout_s, prefix

    def arrive(self, step: int) -> None:
        """Call on every rank before it launches step `step`. Raises PeerLost if a rank is missing."""
        from datetime import timedelta
        try:
            self.store.set(f"{self.prefix}/{step}/{self.rank}", b"1")
            self.store.wait([f"{self.prefix}/{step}/{r}" for r in range(self.world)], timedelta(seconds=self.timeout_s))
        except Exception as exc:  # timeout, or the store's host is gone
            raise PeerLost(f"rank {self.rank}: not every rank of {self.world} arrived for step {step} within {self.timeout_s} s ({type(exc).__name__})") from exc


# ---- device-resident layers -------------------------------------------------------------------

class ColumnParallelTernary:
    """One or several matrices sharing an input (q/k/v, gate/up), rows split across ranks."""

    def __init__(self, packed_list, scales, cols: int, world: int, rank: int, ctx=None):
        import torch
        from . import ops
        self.lins = [ops.TernaryLinear(shard_rows(p, world, rank).contiguous().cuda() if isinstance(p, torch.Tensor)
                                       else torch.from_numpy(np.ascontiguousarray(shard_rows(p, world, rank))).cuda(),
                                       float(s), cols, ctx) for p, s in zip(packed_list, scales)]

    def forward(self, x):
        from . import ops
        return ops.ternary_linear_multi(x, self.lins)


class RowParallelTernary:
    """One matrix with its columns split across ranks; forward returns the full [m, rows] output
    on every rank after an exact integer all-reduce."""

    def __init__(self, packed, scale: float, cols: int, world: int, rank: int, group=None, ctx=None, comm: Optional[TpComm] = None):
        import torch
        from . import ops
        self.comm = comm  # with a TpComm, small batches take the two fused peer-memory kernels instead of NCCL
        sl, self.local_cols = shard_cols(packed, cols, world, rank)
        dev = sl.contiguous().cuda() if isinstance(sl, torch.Tensor) else torch.from_numpy(np.ascontiguousarray(sl)).cuda()
        self.lin = ops.TernaryLinear(dev, float(scale), self.local_cols, ctx)
        self.world, self.group = world, group
        self.rows, self.scale = self.lin.rows, float(scale)
        self.ctx = self.lin.ctx

    def forward(self, x_local):
        """x_local: f32 CUDA [m, cols/world], this rank's column slice of the input."""
        import torch
        import torch.distributed as dist
        from . import _lib
        if x_local.dtype != torch.float32 or x_local.dim() != 2 or x_local.shape[1] != self.local_cols:
            raise ValueError("inner dimension mismatch")
        x_local = x_local.contiguous()
        m = x_local.shape[0]
        lib, h = self.ctx._lib, self.ctx.handle
        st = C.c_void_p(torch.cuda.current_stream().cuda_stream)
        dev = x_local.device
        if (self.comm is not None and self.world > 1 and 0 < m <= self.comm.max_tokens and self.rows % 4 == 0
                and m * self.rows * 4 <= self.comm.partial_bytes):
            return self._forward_fused(x_local, m, st, dev)
        amax = torch.empty(m, dtype=torch.float32, device=dev)
        _lib.check(lib.lbk_absmax_dev(h, C.c_void_p(x_local.data_ptr()), m, self.local_cols, C.c_void_p(amax.data_ptr()), st))
        if self.world > 1:
            dist.all_reduce(amax, op=dist.ReduceOp.MAX, group=self.group)
        kp = (self.local_cols + BLOCK - 1) // BLOCK * BLOCK
        q = torch.empty((m, kp), dtype=torch.int8, device=dev)
        scale = torch.empty(m, dtype=torch.float32, device=dev)
        ssum = torch.empty(m, dtype=torch.int32, device=dev)
        _lib.check(lib.lbk_quantize_acts_amax_dev(h, C.c_void_p(x_local.data_ptr()), m, self.local_cols,
                                                  C.c_void_p(amax.data_ptr()), C.c_void_p(q.data_ptr()),
                                                  C.c_void_p(scale.data_ptr()), C.c_void_p(ssum.data_ptr()), st))
        dots = torch.empty((m, self.rows), dtype=torch.int32, device=dev)
        wp, _k1 = _lib.ptr_array([self.lin.weight.handle.value])
        ip, _k2 = _lib.ptr_array([dots.data_ptr()])
        _lib.check(lib.lbk_ternary_gemm_dev(h, wp, 1, C.c_void_p(q.data_ptr()), None, C.c_void_p(ssum.data_ptr()), m,
                                            None, ip, st))
        if self.world > 1:
            dist.all_reduce(dots, op=dist.ReduceOp.SUM, group=self.group)
        out = torch.empty((m, self.rows), dtype=torch.float32, device=dev)
        _lib.check(lib.lbk_scale_epilogue_dev(h, C.c_void_p(dots.data_ptr()), C.c_void_p(scale.data_ptr()),
                                              C.c_float(self.scale), m, self.rows, C.c_void_p(out.data_ptr()), st))
        return out, dots

    def _forward_fused(self, x_local, m, st, dev):
        """quantise with the all-rank maximum (one kernel) -> int32 partial dots into this rank's
        region -> sum of all ranks' dots + scale (one kernel)."""
        import torch
        from . import _lib
        lib, h, comm = self.ctx._lib, self.ctx.handle, self.comm
        kp = (self.local_cols + BLOCK - 1) // BLOCK * BLOCK
        q = torch.empty((m, kp), dtype=torch.int8, device=dev)
        scale = torch.empty(m, dtype=torch.float32, device=dev)
        ssum = torch.empty(m, dtype=torch.int32, device=dev)
        _lib.check(lib.lbk_tp_quantize(comm.handle, C.c_void_p(x_local.data_ptr()), m, self.local_cols, C.c_void_p(q.data_ptr()),
                                       C.c_void_p(scale.data_ptr()), C.c_void_p(ssum.data_ptr()), st))
        wp, _k1 = _lib.ptr_array([self.lin.weight.handle.value])
        ip, _k2 = _lib.ptr_array([comm.partial_ptr])
        _lib.check(lib.lbk_ternary_gemm_dev(h, wp, 1, C.c_void_p(q.data_ptr()), None, C.c_void_p(ssum.data_ptr()), m, None, ip, st))
        out = torch.empty((m, self.rows), dtype=torch.float32, device=dev)
        dots = torch.empty((m, self.rows), dtype=torch.int32, device=dev)
        _lib.check(lib.lbk_tp_reduce_scale(comm.handle, C.c_void_p(scale.data_ptr()), C.c_float(self.scale), m, self.rows,
                                           C.c_void_p(out.data_ptr()), C.c_void_p(dots.data_ptr()), st))
        return out, dots


# ---- the decoder step, tensor parallel ----------------------------------------------------------

def token_range(m: int, world: int, rank: int):
    """(first token, count) of the ceil(m / world) consecutive token rows rank `rank` owns."""
    mt = (m + world - 1) // world
    t0 = min(rank * mt, m)
    return t0, max(0, min(m - t0, mt))


class _Lin:
    """A packed matrix by handle (a TernaryLinear's, or one owned by a loaded model shard)."""

    def __init__(self, handle: int, rows: int, cols: int, scale: float, keep=None):
        self.handle, self.rows, self.cols, self.scale, self._keep = handle, rows, cols, scale, keep


class TpBitNet:
    """BitNet::forward (crates/lb-model/src/model.rs:305-374) over `world` GPUs, one process each.

    Sharding, as the 70B-shaped configuration states it: q/k/v/gate/up column-parallel (a rank holds
    a row range of the packed matrix = its own attention heads / its slice of the intermediate
    features), o/down row-parallel (a rank holds a 128-aligned column range). The K/V cache holds the
    rank's own KV heads only, and attention runs on the rank's heads. Between the projections the
    activations are exchanged by the library's own peer-memory kernels (lbk_tp_norm_quant,
    lbk_tp_reduce_norm_gather: reduce-scatter of the exact int32 partial dots by token rows, residual
    add + next norm + quantisation on the owner, all-gather of int8 rows); the residual stream lives
    token-sharded. The head is split by vocabulary rows; lbk_tp_argmax picks the greedy token.
    With world == 1 the same calls run without peers (the exchanges are trivial)."""

    def __init__(self, cfg, layers, final_norm, embed, comm: TpComm, ctx, device="cuda"):
        """layers: per layer a dict with _Lin entries q, k, v, o, gate, up, down (already this rank's
        shards) and f32 CUDA tensors input_norm, post_attn_norm (full), attn_sub_norm, ffn_sub_norm
        (this rank's column slices). embed: bf16 CUDA [vocab, hidden] (whole)."""
        import torch
        from .model import rope_tables
        self.cfg, self.layers, self.final_norm, self.embed, self.comm, self.ctx = cfg, layers, final_norm, embed, comm, ctx
        self.world, self.rank, self.device = comm.world, comm.rank, torch.device(device)
        W = self.world
        self.hd = cfg.head_dim()
        if self.hd != 128 or cfg.num_key_value_heads % W or cfg.vocab_size % W or cfg.hidden_size % 128:
            raise ValueError("this model does not divide over the ranks (KV heads, vocabulary) or its head size is not 128")
        self.nh_l, self.kvh_l = cfg.num_attention_heads // W, cfg.num_key_value_heads // W
        self.il = cfg.intermediate_size // W
        self.vl = cfg.vocab_size // W
        cos, sin = rope_tables(cfg)
        self.cos, self.sin = torch.from_numpy(cos).to(self.device), torch.from_numpy(sin).to(self.device)
        lib = ctx._lib
        self.gq, self.gs = int(lib.lbk_tp_gather_q(comm.handle)), int(lib.lbk_tp_gather_scale(comm.handle))
        self.gsum, self.gf = int(lib.lbk_tp_gather_sum(comm.handle)), int(lib.lbk_tp_gather_f32(comm.handle))
        self._bufs = {}

    # ---- construction ----------------------------------------------------------------------------
    @classmethod
    def from_tensors(cls, cfg, tensors, comm: TpComm, ctx, device="cuda"):
        """Shards a full checkpoint dict (names as in model.lbt.safetensors; CPU or CUDA tensors)."""
        import torch
        from . import ops
        W, r = comm.world, comm.rank
        H, I = cfg.hidden_size, cfg.intermediate_size
        nhd = cfg.num_attention_heads * cfg.head_dim()
        dev = torch.device(device)

        def col(name, cols):  # column-parallel: a row range
            qw = tensors[f"{name}.qweight"]
            lin = ops.TernaryLinear(shard_rows(qw, W, r).contiguous().to(dev), float(tensors[f"{name}.wscale"].reshape(-1)[0]), cols, ctx)
            return _Lin(lin.weight.handle.value, lin.rows, cols, lin.scale, lin)

        def row(name, cols):  # row-parallel: a column range
            sl, lc = shard_cols(tensors[f"{name}.qweight"], cols, W, r)
            lin = ops.TernaryLinear(sl.contiguous().to(dev), float(tensors[f"{name}.wscale"].reshape(-1)[0]), lc, ctx)
            return _Lin(lin.weight.handle.value, lin.rows, lc, lin.scale, lin)

        layers = []
        for i in range(cfg.num_hidden_layers):
            p = f"model.layers.{i}"
            vec = lambda n: tensors[f"{p}.{n}.weight"].to(dev).float().contiguous()
            sub_a, sub_f = vec("self_attn.attn_sub_norm"), vec("mlp.ffn_sub_norm")
            layers.append(dict(q=col(f"{p}.self_attn.q_proj", H), k=col(f"{p}.self_attn.k_proj", H), v=col(f"{p}.self_attn.v_proj", H),
                               o=row(f"{p}.self_attn.o_proj", nhd), gate=col(f"{p}.mlp.gate_proj", H), up=col(f"{p}.mlp.up_proj", H),
                               down=row(f"{p}.mlp.down_proj", I), input_norm=vec("input_layernorm"), post_attn_norm=vec("post_attention_layernorm"),
                               attn_sub_norm=sub_a[r * nhd // W:(r + 1) * nhd // W].contiguous(), ffn_sub_norm=sub_f[r * I // W:(r + 1) * I // W].contiguous()))
        return cls(cfg, layers, tensors["model.norm.weight"].to(dev).float().contiguous(), tensors["model.embed_tokens.weight"].to(dev).contiguous(),
                   comm, ctx, device)

    @classmethod
    def random_init(cls, cfg, seed: int, comm: TpComm, ctx, device="cuda", p_zero: float = 0.4):
        """Random-init weights of the given architecture, generated on the device and kept as this
        rank's shards only: i.i.d. ternary codes with P(0) = p_zero and P(-1) = P(+1), norm gains near 1,
        bf16 embedding N(0, 0.02). Every tensor has its own seed, the same on every rank, so that the
        ranks hold slices of one model; the full tensor exists only while it is sliced."""
        import torch
        from . import ops
        from .pack import row_bytes as _rb
        W, r = comm.world, comm.rank
        H, I = cfg.hidden_size, cfg.intermediate_size
        nhd = cfg.num_attention_heads * cfg.head_dim()
        kvd = cfg.num_key_value_heads * cfg.head_dim()
        dev = torch.device(device)
        scale = float(np.float32(1.0) / np.float32(0.02 * np.sqrt(2.0 / np.pi)))  # 1 / mean|N(0, 0.02)|

        def packed(rows, cols, tseed):
            g = torch.Generator(device=dev).manual_seed(tseed)
            lo = int(round((1.0 - p_zero) / 2 * 1000))
            v = torch.randint(0, 1000, (4, rows, _rb(cols)), dtype=torch.int16, generator=g, device=dev)
            codes = (v >= lo).to(torch.uint8) + (v >= 1000 - lo).to(torch.uint8)
            return codes[0] | (codes[1] << 2) | (codes[2] << 4) | (codes[3] << 6)

        def col(rows, cols, tseed):
            lin = ops.TernaryLinear(shard_rows(packed(rows, cols, tseed), W, r).contiguous(), scale, cols, ctx)
            return _Lin(lin.weight.handle.value, lin.rows, cols, lin.scale, lin)

        def row(rows, cols, tseed):
            sl, lc = shard_cols(packed(rows, cols, tseed), cols, W, r)
            lin = ops.TernaryLinear(sl.contiguous(), scale, lc, ctx)
            return _Lin(lin.weight.handle.value, lin.rows, lc, lin.scale, lin)

        layers = []
        for i in range(cfg.num_hidden_layers):
            s0 = seed * 100003 + i * 16
            g = torch.Generator(device=dev).manual_seed(s0 + 15)
            gain = lambda n: (1.0 + 0.05 * torch.randn(n, generator=g, device=dev)).float()
            inp, post, sub_a, sub_f = gain(H), gain(H), gain(nhd), gain(I)
            layers.append(dict(q=col(nhd, H, s0), k=col(kvd, H, s0 + 1), v=col(kvd, H, s0 + 2), o=row(H, nhd, s0 + 3),
                               gate=col(I, H, s0 + 4), up=col(I, H, s0 + 5), down=row(H, I, s0 + 6), input_norm=inp, post_attn_norm=post,
                               attn_sub_norm=sub_a[r * nhd // W:(r + 1) * nhd // W].contiguous(), ffn_sub_norm=sub_f[r * I // W:(r + 1) * I // W].contiguous()))
        g = torch.Generator(device=dev).manual_seed(seed * 100003 + 99991)
        final = (1.0 + 0.05 * torch.randn(H, generator=g, device=dev)).float()
        embed = torch.empty((cfg.vocab_size, H), dtype=torch.bfloat16, device=dev)
        step = 8192
        for v0 in range(0, cfg.vocab_size, step):  # in slabs: the f32 draw of the whole table would be twice its size
            n = min(step, cfg.vocab_size - v0)
            embed[v0:v0 + n] = (0.02 * torch.randn(n, H, generator=g, device=dev)).to(torch.bfloat16)
        net = cls(cfg, layers, final, embed, comm, ctx, device)
        net._packed_for_check = packed
        return net

    @classmethod
    def from_native(cls, native, comm: TpComm, device="cuda"):
        """Wraps a shard loaded by lbk_model_load_shard (model.NativeBitNet with rank / world): the packed
        matrices stay where the loader put them; norm gains and the embedding are viewed in place."""
        import torch
        cfg, lib, W, r = native.cfg, native._lib, comm.world, comm.rank
        if (native.rank, native.world) != (r, W):
            raise ValueError("the model shard and the communicator disagree on rank / world")
        H, I, nhd = cfg.hidden_size, cfg.intermediate_size, cfg.num_attention_heads * cfg.head_dim()

        def lin(layer, name):
            h = native.linear_handle(layer, name)
            return _Lin(h, int(lib.lbk_weight_rows(h)), int(lib.lbk_weight_cols(h)), float(lib.lbk_weight_scale(h)), native)

        layers = []
        for i in range(cfg.num_hidden_layers):
            layers.append(dict(q=lin(i, "q"), k=lin(i, "k"), v=lin(i, "v"), o=lin(i, "o"), gate=lin(i, "gate"), up=lin(i, "up"), down=lin(i, "down"),
                               input_norm=_DevView(native.norm_ptr(i, "input_norm"), H), post_attn_norm=_DevView(native.norm_ptr(i, "post_attn_norm"), H),
                               attn_sub_norm=_DevView(native.norm_ptr(i, "attn_sub_norm") + 4 * (r * nhd // W), nhd // W),
                               ffn_sub_norm=_DevView(native.norm_ptr(i, "ffn_sub_norm") + 4 * (r * I // W), I // W)))
        return cls(cfg, layers, _DevView(native.norm_ptr(0, "final_norm"), H), _DevView(int(lib.lbk_model_embedding(native.handle)), cfg.vocab_size * H, 2),
                   comm, native.ctx, device)

    # ---- state -----------------------------------------------------------------------------------
    def new_cache(self, b: int, cap: int):
        """K/V rows of this rank's KV heads: bf16 [layers][b][kv_heads / world][cap][128]; one position per sequence."""
        import torch
        cfg = self.cfg
        if cap < 1 or cap > cfg.max_position_embeddings:
            raise ValueError(f"capacity {cap} is outside 1..max_position_embeddings ({cfg.max_position_embeddings})")
        shape = (cfg.num_hidden_layers, b, self.kvh_l, cap, self.hd)
        return dict(k=torch.zeros(shape, dtype=torch.bfloat16, device=self.device), v=torch.zeros(shape, dtype=torch.bfloat16, device=self.device),
                    pos=torch.zeros(b, dtype=torch.int32, device=self.device), b=b, cap=cap, host_len=[0] * b)

    def _buf(self, name, shape, dtype=None):
        import torch
        key = (name, tuple(shape), dtype or torch.float32)
        if key not in self._bufs:
            self._bufs[key] = torch.zeros(shape, dtype=dtype or torch.float32, device=self.device)
        return self._bufs[key]

    # ---- one step ----------------------------------------------------------------------------------
    def forward(self, tokens, cache, prompt: bool = False, trace=None):
        """tokens: int32 CUDA [m]. prompt=False: one new token for each of the cache's m sequences.
        prompt=True: m consecutive tokens of sequence 0 (a cache made for one sequence). Returns
        (logits of this rank's vocabulary slice: [m, vocab / world], or [1, vocab / world] for the last
        prompt token; greedy tokens int32 [m] or [1], the same on every rank) and advances the cache.
        trace: a list that receives (operation name, CUDA event recorded after it) pairs, for a per-operation
        time breakdown of an eager step (not for use under graph capture)."""
        import torch
        from . import _lib
        from .model import attention_splits
        cfg, lib, h, comm = self.cfg, self.ctx._lib, self.ctx.handle, self.comm
        m = int(tokens.shape[0])
        if (not prompt and m != cache["b"]) or (prompt and cache["b"] != 1):
            raise ValueError("token count and cache do not match")
        need = m if prompt else 1
        for used in cache["host_len"]:
            if used + need > cache["cap"]:  # model.rs:309
                raise ValueError(f"the cache is full: {used} of {cache['cap']} positions are used, {need} more do not fit")
        H, I, hd, eps = cfg.hidden_size, cfg.intermediate_size, self.hd, cfg.rms_norm_eps
        nh_l, kvh_l, il, L = self.nh_l, self.kvh_l, self.il, cfg.num_hidden_layers
        st = C.c_void_p(torch.cuda.current_stream().cuda_stream)
        P = lambda t: C.c_void_p(t.data_ptr() if hasattr(t, "data_ptr") else int(t))
        chk = _lib.check
        t0, cnt = token_range(m, self.world, self.rank)
        mt = (m + self.world - 1) // self.world
        xres = self._buf("xres", (max(mt, 1), H))
        q = self._buf("q", (m, nh_l * hd)); k = self._buf("k", (m, kvh_l * hd)); v = self._buf("v", (m, kvh_l * hd))
        attn = self._buf("attn", (m, nh_l * hd))
        g = self._buf("g", (m, il)); u = self._buf("u", (m, il))
        q8 = self._buf("q8", (m, max(nh_l * hd, il)), torch.int8)
        qs, qsum = self._buf("qs", (m,)), self._buf("qsum", (m,), torch.int32)
        splits = attention_splits(cache["cap"])  # an upper bound: the batched kernel takes fewer, longer slices when the batch fills the GPU
        scratch = self._buf("attn_part", (m * nh_l * splits * (hd + 4),))
        counters = self._buf("attn_counters", (m * kvh_l,), torch.int32)
        rows_out = 1 if prompt else m
        logits = self._buf("logits", (rows_out, self.vl))
        idx, nxt = self._buf("idx", (rows_out,), torch.int32), self._buf("next", (rows_out,), torch.int32)

        def mark(name):
            if trace is not None:
                ev = torch.cuda.Event(enable_timing=True)
                ev.record()
                trace.append((name, ev))

        def gemm(qp, sp, sump, lins, outs, iouts):
            wp, k1 = _lib.ptr_array([l.handle for l in lins])
            op, k2 = _lib.ptr_array([o.data_ptr() for o in outs]) if outs else (None, None)
            ip, k3 = _lib.ptr_array(iouts) if iouts else (None, None)
            chk(lib.lbk_ternary_gemm_dev(h, wp, len(lins), C.c_void_p(qp), C.c_void_p(sp) if sp else None, C.c_void_p(sump), m, op, ip, st))

        # From 256 token rows on (a prompt pass) and with four ranks or more, a row-parallel projection stores its
        # partial dots into the token owners' regions from its own epilogue (lbk_tp_gemm_scatter) and the exchange
        # kernel adds up what arrived (measured at four ranks: exchange 19.4 -> 11.2 ms per 2048-token pass, the two
        # projections 9.3 -> 16.8 ms, the pass 56.3 -> 55.4 ms; at two ranks the projections lose more than the
        # exchange gains). Decode batches keep the GEMM that may split K over idle SMs and the exchange that pulls.
        scatter = comm.world >= 4 and m >= 256
        sflag = 4 if scatter else 0  # LBK_TP_SCATTERED

        def row_parallel_gemm(lin):
            if scatter:
                chk(lib.lbk_tp_gemm_scatter(comm.handle, lin.handle, C.c_void_p(q8.data_ptr()), C.c_void_p(qsum.data_ptr()), m, st))
            else:
                gemm(q8.data_ptr(), None, qsum.data_ptr(), [lin], None, [comm.partial_ptr])

        def reduce_norm_gather(flags, ascale, wscale, gain):
            chk(lib.lbk_tp_reduce_norm_gather(comm.handle, flags, P(ascale) if ascale is not None else None, C.c_float(wscale), P(xres), P(gain),
                                              C.c_float(eps), m, H, None, st))

        mark("start")
        if cnt:
            chk(lib.lbk_embed_bf16(h, P(self.embed), C.c_void_p(tokens.data_ptr() + 4 * t0), cnt, H, P(xres), st))
        reduce_norm_gather(1, None, 1.0, self.layers[0]["input_norm"])  # LBK_TP_NO_REDUCE
        mark("embed + norm + gather")
        for li, l in enumerate(self.layers):
            gemm(self.gq, self.gs, self.gsum, [l["q"], l["k"], l["v"]], [q, k, v], None)
            mark("q/k/v GEMM")
            kc, vc = cache["k"][li], cache["v"][li]
            if prompt:
                chk(lib.lbk_rope_kv_append_rows(h, P(q), P(k), P(v), P(self.cos), P(self.sin), P(cache["pos"]), m, nh_l, kvh_l, hd, cache["cap"], 0,
                                                P(kc), P(vc), st))
                chk(lib.lbk_attn_prefill(h, P(q), P(kc), P(vc), P(cache["pos"]), m, nh_l, kvh_l, hd, cache["cap"], 0, P(attn), st))
            elif lib.lbk_attn_decode_fused_supported(nh_l, kvh_l, hd, splits):
                chk(lib.lbk_attn_decode_fused_seq(h, P(q), P(k), P(v), P(self.cos), P(self.sin), P(cache["pos"]), m, nh_l, kvh_l, hd, cache["cap"],
                                                  splits, P(kc), P(vc), P(scratch), P(counters), P(attn), st))
            else:
                chk(lib.lbk_rope_kv_append_seq(h, P(q), P(k), P(v), P(self.cos), P(self.sin), P(cache["pos"]), m, nh_l, kvh_l, hd, cache["cap"],
                                               P(kc), P(vc), st))
                chk(lib.lbk_attn_decode_seq(h, P(q), P(kc), P(vc), P(cache["pos"]), m, nh_l, kvh_l, hd, cache["cap"], splits, P(scratch), P(attn), st))
            mark("attention (RoPE, K/V append, softmax)")
            chk(lib.lbk_tp_norm_quant(comm.handle, 1, P(attn), None, P(l["attn_sub_norm"]), m, nh_l * hd, cfg.num_attention_heads * hd, C.c_float(eps),
                                      P(q8), P(qs), P(qsum), st))
            mark("sub-norm + quantise (statistics exchange)")
            row_parallel_gemm(l["o"])
            mark("o GEMM")
            reduce_norm_gather(sflag, qs, l["o"].scale, l["post_attn_norm"])
            mark("reduce-scatter + residual + norm + all-gather")
            gemm(self.gq, self.gs, self.gsum, [l["gate"], l["up"]], [g, u], None)
            mark("gate/up GEMM")
            chk(lib.lbk_tp_norm_quant(comm.handle, 3, P(g), P(u), P(l["ffn_sub_norm"]), m, il, I, C.c_float(eps), P(q8), P(qs), P(qsum), st))
            mark("sub-norm + quantise (statistics exchange)")
            row_parallel_gemm(l["down"])
            mark("down GEMM")
            last = li + 1 == L
            reduce_norm_gather((2 if last else 0) | sflag, qs, l["down"].scale, self.final_norm if last else self.layers[li + 1]["input_norm"])
            mark("reduce-scatter + residual + norm + all-gather")
        # the head: this rank's vocabulary rows of the tied embedding (model.rs:370-373), then the greedy token
        head_in = self.gf + (4 * H * (m - 1) if prompt else 0)
        chk(lib.lbk_bf16_linear(h, C.c_void_p(head_in), rows_out, C.c_void_p(_ptr(self.embed) + 2 * H * self.vl * self.rank), self.vl, H, P(logits), st))
        chk(lib.lbk_argmax(h, P(logits), rows_out, self.vl, P(idx), st))
        chk(lib.lbk_tp_argmax(comm.handle, P(logits), P(idx), rows_out, self.vl, P(nxt), st))
        if prompt:
            cache["pos"].add_(m)
        else:
            chk(lib.lbk_advance_pos_seq(h, P(cache["pos"]), None, m, st))
        mark("head + greedy token")
        cache["host_len"] = [x + need for x in cache["host_len"]]
        return logits, nxt


class _DevView:
    """A device address with an element count (memory owned by a loaded model)."""

    def __init__(self, ptr: int, n: int, elem_bytes: int = 4):
        self.ptr, self.n, self.elem_bytes = int(ptr), n, elem_bytes

    def data_ptr(self) -> int:
        return self.ptr


def _ptr(t) -> int:
    return int(t.data_ptr())
