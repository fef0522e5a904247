"""Expert-parallel host logic on CPU: two gloo ranks, no GPU.

Checks (a) the handle exchange of ``MoELayer.ep_connect`` delivers every rank's
blob in rank order, and (b) the row layout rules the device implements
(restated in ``omega_ai_b200/ep_layout.py``): simulated dispatch fills every
owner's buffer without overlap, grouped by expert, ordered by (source rank,
flat pick index), and a pull-style combine with identity experts returns the
gate-weighted sum of the token itself.
"""
import os
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, q):
    try:
        sys.path.insert(0, ROOT)
        os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
        dist.init_process_group("gloo", rank=rank, world_size=world)
        from omega_ai_b200 import ep_layout as L
        from omega_ai_b200 import native
        from omega_ai_b200.layer import MoELayer
        from oracle import ref

        # (a) blob exchange through the real ep_connect, with the native calls stubbed out
        class Fake(MoELayer):
            def __init__(self):
                self.world, self.rank, self.got = world, rank, None

            def ep_export(self):
                return bytes([rank]) * native.EP_BLOB_BYTES

            def ep_import(self, blobs):
                self.got = blobs

            def __del__(self):
                pass

        torch.cuda.synchronize = lambda *a, **k: None  # no GPU here
        f = Fake()
        f.ep_connect()
        assert [b[0] for b in f.got] == list(range(world)) and all(len(b) == native.EP_BLOB_BYTES for b in f.got)

        # (b) layout rules
        E, k, d, T_all = 8, 2, 16, 301
        e_local = E // world
        lo, hi = L.shard_tokens(T_all, world, rank)
        rng = np.random.Generator(np.random.Philox(key=5))
        x_all = rng.standard_normal((T_all, d), dtype=np.float32)
        w_r = (0.5 * rng.standard_normal((E, d))).astype(np.float32)
        x = x_all[lo:hi]
        idx, gate = ref.topk_gate(ref.router_logits(x, w_r), k)
        counts, offsets, perm, pos = ref.histogram_permute(idx, E)
        gathered = [None] * world
        dist.all_gather_object(gathered, counts)
        counts_all = np.stack(gathered)
        base = L.dst_base(counts_all, rank, e_local)
        # row of every pick in its owner's buffer
        flat = idx.reshape(-1)
        row = base[flat] + (pos - offsets[flat])
        owner = flat // e_local
        # "dispatch": every rank publishes (owner, row, payload); owners assemble their buffers
        sends = [None] * world
        dist.all_gather_object(sends, (owner, row, np.repeat(x, k, axis=0), np.full(flat.size, rank), np.arange(flat.size)))
        cap = L.rows_needed(counts_all, e_local)
        buf = np.full((cap, d), np.nan, np.float32)
        tag = np.full((cap, 2), -1, np.int64)
        for (ow, rw, payload, src, f_idx) in sends:
            m = ow == rank
            assert (tag[rw[m], 0] == -1).all(), "two picks landed on one row"
            buf[rw[m]] = payload[m]
            tag[rw[m], 0], tag[rw[m], 1] = src[m], f_idx[m]
        ex_counts, ex_poff = L.owner_layout(counts_all, rank, e_local)
        for le in range(e_local):
            seg = tag[ex_poff[le]:ex_poff[le] + ex_counts[le]]
            assert (seg[:, 0] >= 0).all()
            key = seg[:, 0] * 10**6 + seg[:, 1]
            assert (np.diff(key) > 0).all(), "rows not ordered by (source rank, flat index)"
            assert (tag[ex_poff[le] + ex_counts[le]:ex_poff[le + 1], 0] == -1).all()  # padding untouched
            assert ex_poff[le] % L.ROW_ALIGN == 0
        # "combine" by pulling rows back from the owners (identity experts)
        bufs = [None] * world
        dist.all_gather_object(bufs, buf)
        y = np.zeros_like(x)
        for t in range(x.shape[0]):
            for j in range(k):
                fidx = t * k + j
                y[t] += gate[t, j] * bufs[owner[fidx]][row[fidx]]
        np.testing.assert_allclose(y, x * gate.sum(1, keepdims=True), rtol=1e-5, atol=1e-6)
        dist.barrier()
        dist.destroy_process_group()
        q.put((rank, "ok"))
    except Exception as e:  # noqa: BLE001
        import traceback

        q.put((rank, "FAIL " + traceback.format_exc()))


@pytest.mark.parametrize("world", [2, 4])
def test_ep_host_logic_gloo(world):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29600 + world
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = [q.get(timeout=120) for _ in procs]
    for p in procs:
        p.join(timeout=30)
    assert all(msg == "ok" for _, msg in results), results


def test_shard_tokens_cover_the_batch():
    sys.path.insert(0, ROOT)
    from omega_ai_b200 import ep_layout as L

    for T in (0, 1, 7, 16384, 16385):
        for W in (1, 2, 4, 8):
            spans = [L.shard_tokens(T, W, r) for r in range(W)]
            assert spans[0][0] == 0 and spans[-1][1] == T
            assert all(spans[i][1] == spans[i + 1][0] for i in range(W - 1))


def test_refusal_rule_and_capacity():
    """A step whose padded rows exceed any owner's capacity is refused on every rank alike: the layout rule gives
    REFUSED_BASE for every expert, so every derived row position is negative and no row moves."""
    sys.path.insert(0, ROOT)
    from omega_ai_b200 import ep_layout as L

    e_local = 2
    counts_all = np.array([[100, 3, 0, 40], [60, 0, 0, 500]], np.int32)  # [source rank, expert]
    need = L.rows_needed(counts_all, e_local)
    assert need == 640  # owner 1: expert 2 empty -> 0 rows, expert 3: 540 -> 640; owner 0: 160 -> 256, 3 -> 128
    cap_ok = L.rows_capacity(540, e_local)   # recv_rows_max = 540 rows: (5 + 2) * 128
    assert cap_ok == 896 and not L.step_refused(counts_all, e_local, cap_ok)
    base = L.dst_base(counts_all, 1, e_local, cap_ok)
    assert base.tolist() == [100, 256 + 3, 0, 0 + 40]
    cap_small = L.rows_capacity(100, e_local)  # (1 + 2) * 128 = 384 < 640
    assert L.step_refused(counts_all, e_local, cap_small)
    for r in range(2):
        b = L.dst_base(counts_all, r, e_local, cap_small)
        assert (b == L.REFUSED_BASE).all()
        # any position derived from a refused base is negative whatever the in-expert offset (< 2^30)
        assert (b.astype(np.int64) + counts_all.sum() < 0).all()


def _rendezvous_worker(rank, world, port, q, absent):
    try:
        sys.path.insert(0, ROOT)
        import datetime

        from omega_ai_b200 import native
        from omega_ai_b200.layer import MoELayer

        store = dist.TCPStore("127.0.0.1", port, world, is_master=(rank == 0),
                              timeout=datetime.timedelta(seconds=20), wait_for_workers=False)

        class Fake(MoELayer):
            def __init__(self):
                self.world, self.rank, self.got = world, rank, None

            def ep_export(self):
                return bytes([rank]) * native.EP_BLOB_BYTES

            def ep_import(self, blobs):
                self.got = blobs

            def __del__(self):
                pass

        torch.cuda.synchronize = lambda *a, **k: None  # no GPU here
        if rank in absent:
            # this rank never posts its handles: it stays alive (the store must outlive the others' deadline when
            # it is the master) and leaves quietly
            import time
            time.sleep(4.0)
            q.put((rank, "absent"))
            return
        f = Fake()
        try:
            f.ep_connect(store=store, timeout_s=1.5)
            assert [b[0] for b in f.got] == list(range(world))
            q.put((rank, "ok"))
        except native.OmoeError as e:
            q.put((rank, f"comm-error code={e.code} {e}"))
        if rank == 0:
            import time
            time.sleep(1.0)  # the master store stays up until the other ranks have read what they need
    except Exception:  # noqa: BLE001
        import traceback

        q.put((rank, "FAIL " + traceback.format_exc()))


@pytest.mark.parametrize("absent", [(), (1,)])
def test_rendezvous_with_deadline(absent):
    """Failure detection on the host: with a store, ep_connect is a rendezvous with a deadline.  All ranks present:
    handles arrive in rank order.  Rank 1 never posts: rank 0 gets OMOE_ERR_COMM naming rank 1 after the deadline
    instead of waiting forever."""
    world = 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29650 + len(absent)
    procs = [ctx.Process(target=_rendezvous_worker, args=(r, world, port, q, absent)) for r in range(world)]
    for p in procs:
        p.start()
    results = dict(q.get(timeout=120) for _ in procs)
    for p in procs:
        p.join(timeout=30)
    if not absent:
        assert results == {0: "ok", 1: "ok"}, results
    else:
        assert results[1] == "absent"
        assert results[0].startswith("comm-error code=-7") and "rank 1 did not post" in results[0], results
