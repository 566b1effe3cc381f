"""Host-side logic of the tensor-parallel path on CPU: two gloo ranks shard a packed matrix with
the package's slicing helpers, all-reduce exactly as the GPU layers do (MAX of the per-token
maxima, integer SUM of the partial dots), and must reproduce the unsharded result bit for bit.
The arithmetic on each rank is the CPU oracle (this is a test; the product path runs the CUDA
kernels), the collectives and the slicing are the real ones."""
import os
import socket
import sys
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parent.parent


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, q_out):
    sys.path.insert(0, str(ROOT))
    import torch
    import torch.distributed as dist
    from lemonade_burn_b200 import tp
    from oracle import oracle as o
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        rng = np.random.default_rng(7)
        rows, cols, m = 48, 1024, 5
        t = rng.choice(np.array([-1, 0, 1], dtype=np.int8), size=(rows, cols), p=[0.3, 0.4, 0.3])
        packed = o.pack_matrix(t)
        x = rng.standard_normal((m, cols)).astype(np.float32)
        x[1, 700] = 9.5  # the row maximum of token 1 lives in rank 1's slice
        wscale = np.float32(41.5)
        # reference: unsharded
        q, s, ssum = o.quantize_acts(x)
        want_i = o.ternary_gemm_i32(packed, cols, q, ssum)
        want_f = o.ternary_gemm(packed, cols, wscale, q, s, ssum)
        # row-parallel: column slices
        sl, lc = tp.shard_cols(packed, cols, world, rank)
        xl = x[:, rank * lc:(rank + 1) * lc]
        amax = torch.from_numpy(np.abs(xl).max(axis=1).astype(np.float32))
        dist.all_reduce(amax, op=dist.ReduceOp.MAX)
        scale = (np.float32(127.0) / np.maximum(amax.numpy(), np.float32(1e-5))).astype(np.float32)
        ql = np.clip(np.rint(xl * scale[:, None]), -128, 127).astype(np.int8)
        lsum = ql.astype(np.int32).sum(axis=1).astype(np.int32)
        part = torch.from_numpy(o.ternary_gemm_i32(np.ascontiguousarray(sl), lc, ql, lsum))
        dist.all_reduce(part, op=dist.ReduceOp.SUM)
        got_i = part.numpy()
        inv = (np.float32(1.0) / (scale * wscale)).astype(np.float32)
        got_f = (got_i.astype(np.float32) * inv[:, None]).astype(np.float32)
        ok_row = np.array_equal(got_i, want_i) and np.array_equal(got_f.view(np.uint32), want_f.view(np.uint32)) \
            and np.array_equal(scale.view(np.uint32), s.view(np.uint32))
        # column-parallel: row slices, gathered
        rs = tp.shard_rows(packed, world, rank)
        loc = torch.from_numpy(o.ternary_gemm_i32(np.ascontiguousarray(rs), cols, q, ssum))
        parts = [torch.empty_like(loc) for _ in range(world)]
        dist.all_gather(parts, loc)
        ok_col = np.array_equal(torch.cat(parts, dim=1).numpy(), want_i)
        q_out.put((rank, bool(ok_row), bool(ok_col)))
    finally:
        dist.destroy_process_group()


def test_two_rank_sharding_is_exact():
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = [q.get(timeout=120) for _ in procs]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for rank, ok_row, ok_col in res:
        assert ok_row, f"rank {rank}: row-parallel result differs from the unsharded one"
        assert ok_col, f"rank {rank}: column-parallel result differs from the unsharded one"


def test_shard_helpers_reject_bad_cuts():
    from lemonade_burn_b200 import tp
    packed = np.zeros((6, 96), dtype=np.uint8)  # 384 columns
    with pytest.raises(ValueError, match="128-column blocks"):
        tp.shard_cols(packed, 384, 2, 0)       # 192 columns per rank: not block aligned
    with pytest.raises(ValueError, match="do not divide"):
        tp.shard_rows(packed, 4, 0)
    sl, lc = tp.shard_cols(packed, 384, 3, 1)
    assert lc == 128 and sl.shape == (6, 32)


def _token_sharded_worker(rank, world, port, q_out):
    """The token-sharded form of a row-parallel layer on CPU ranks: int32 partial dots of the column
    slices, reduce-scatter by token rows (here: integer all-reduce, then the owner keeps its rows; and
    the scattering form, where every source rank delivers the owner's rows into the owner's buffer),
    scale epilogue + residual on the owner, all-gather of the owners' rows. Uneven ownership (5 tokens
    over 2 ranks, 3 over 4 with an empty rank) included."""
    sys.path.insert(0, str(ROOT))
    import torch
    import torch.distributed as dist
    from lemonade_burn_b200 import tp
    from oracle import oracle as o
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        ok = True
        for m in (5, 3, 1):
            rng = np.random.default_rng(11 + m)
            rows, cols = 256, 512 * world
            t = rng.choice(np.array([-1, 0, 1], dtype=np.int8), size=(rows, cols), p=[0.3, 0.4, 0.3])
            packed = o.pack_matrix(t)
            x = rng.standard_normal((m, cols)).astype(np.float32)
            resid = rng.standard_normal((m, rows)).astype(np.float32)
            wscale = np.float32(33.25)
            q, s, ssum = o.quantize_acts(x)
            want = (resid + o.ternary_gemm(packed, cols, wscale, q, s, ssum)).astype(np.float32)
            sl, lc = tp.shard_cols(packed, cols, world, rank)
            ql = np.ascontiguousarray(q[:, rank * lc:(rank + 1) * lc])          # every rank quantises with the whole row's scale
            lsum = ql.astype(np.int32).sum(axis=1).astype(np.int32)
            part = torch.from_numpy(o.ternary_gemm_i32(np.ascontiguousarray(sl), lc, ql, lsum))
            own_part = part.clone()
            dist.all_reduce(part, op=dist.ReduceOp.SUM)
            t0, cnt = tp.token_range(m, world, rank)
            # the scattering form of the same exchange (the projection's epilogue stores a token row's dots
            # straight into its owner's buffer, laid out [source rank][token of the owner][row]): what an
            # owner finds in its buffer, added up over the source ranks in any order, is the all-reduce's rows
            mt_s = (m + world - 1) // world
            send = torch.zeros((world, mt_s, rows), dtype=torch.int32)
            for owner in range(world):
                o0, oc = tp.token_range(m, world, owner)
                send[owner, :oc] = own_part[o0:o0 + oc]
            got = [torch.empty_like(send) for _ in range(world)]
            dist.all_gather(got, send)
            arrived = torch.stack([got[src][rank] for src in range(world)])  # [source rank][token][row] in MY buffer
            summed = arrived.flip(0).sum(dim=0, dtype=torch.int32)
            ok = ok and torch.equal(summed[:cnt], part[t0:t0 + cnt])
            inv = (np.float32(1.0) / (s * wscale)).astype(np.float32)
            mine = (resid[t0:t0 + cnt] + part.numpy()[t0:t0 + cnt].astype(np.float32) * inv[t0:t0 + cnt, None]).astype(np.float32)
            mt = (m + world - 1) // world
            pad = np.zeros((mt, rows), np.float32)
            pad[:cnt] = mine
            parts = [torch.empty((mt, rows)) for _ in range(world)]
            dist.all_gather(parts, torch.from_numpy(pad))
            full = torch.cat(parts, dim=0).numpy()[:m]
            ok = ok and np.array_equal(full.view(np.uint32), want.view(np.uint32))
            spans = [tp.token_range(m, world, r) for r in range(world)]
            ok = ok and sum(c for _, c in spans) == m and all(a + c == spans[i + 1][0] or spans[i + 1][1] == 0 for i, (a, c) in enumerate(spans[:-1]))
        q_out.put((rank, bool(ok)))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4])
def test_token_sharded_exchange_is_exact(world):
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_token_sharded_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = [q.get(timeout=120) for _ in procs]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert all(ok for _, ok in res), res


def _leaving_worker(rank, world, port, q_out):
    sys.path.insert(0, str(ROOT))
    import time
    from datetime import timedelta
    import torch.distributed as dist
    from lemonade_burn_b200 import tp
    store = dist.TCPStore("127.0.0.1", port, world, is_master=(rank == 0), timeout=timedelta(seconds=20))
    guard = tp.PeerGuard(store, world, rank, timeout_s=1.5)
    done = 0
    try:
        for step in range(4):
            if rank == 1 and step == 2:
                q_out.put((rank, "left", done))      # leaves between steps, nothing in flight
                return
            guard.arrive(step)
            done += 1                                  # a step would be launched here
        q_out.put((rank, "finished", done))
    except tp.PeerLost as exc:
        q_out.put((rank, "peer lost", done))
        time.sleep(0.2)


def test_a_rank_that_leaves_between_steps_is_an_error_not_a_hang():
    """Failure detection on the host: rank 1 of 2 leaves after two steps; rank 0 must find out before
    launching the third (PeerLost within the guard's timeout), not wait forever."""
    import time
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_leaving_worker, args=(r, 2, port, q)) for r in range(2)]
    t0 = time.time()
    for p in procs:
        p.start()
    res = dict((r, (what, n)) for r, what, n in [q.get(timeout=60) for _ in procs])
    for p in procs:
        p.join(timeout=30)
        assert p.exitcode == 0
    assert res[1] == ("left", 2)
    assert res[0] == ("peer lost", 2)
    assert time.time() - t0 < 45
