"""Host-side logic of the expert-parallel exchange on CPU: the numpy plan (what tf_ep_pack computes) driven
through real all-to-all collectives with the gloo backend, world size 2 and 4."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _fake_expert(rows, expert_global):
    """Stand-in for an expert FFN: deterministic, different per expert."""
    return rows * (1.0 + 0.125 * expert_global[:, None]) + expert_global[:, None]


def _worker(rank, world, port, fixed, T, K, E, D, out_dir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    import sys
    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    from turbo_fieldfare_b200.ep import EMPTY_SLOT, plan_dispatch
    rng = np.random.default_rng(100 + rank)
    x = rng.standard_normal((T, D)).astype(np.float32)
    idx = np.stack([rng.permutation(E)[:K] for _ in range(T)]).astype(np.uint32)
    w = rng.dirichlet(np.ones(K), size=T).astype(np.float32)
    epr = E // world
    cap = T * K if fixed else 0
    send_token, send_eloc, inverse, send_counts = plan_dispatch(idx, epr, world, cap)
    slots = send_token.size
    send_rows = np.zeros((slots, D), dtype=np.float32)
    valid = send_token >= 0
    send_rows[valid] = x[send_token[valid]]
    if fixed:
        recv_ids = torch.empty(slots, dtype=torch.int64)
        recv_rows = torch.empty(slots, D)
        dist.all_to_all_single(recv_ids, torch.from_numpy(send_eloc.astype(np.int64)))
        dist.all_to_all_single(recv_rows, torch.from_numpy(send_rows))
        in_splits = out_splits = None
    else:
        sc = torch.from_numpy(send_counts.copy())
        rc = torch.empty_like(sc)
        dist.all_to_all_single(rc, sc)
        in_splits, out_splits = [int(v) for v in sc], [int(v) for v in rc]
        recv_ids = torch.empty(sum(out_splits), dtype=torch.int64)
        recv_rows = torch.empty(sum(out_splits), D)
        dist.all_to_all_single(recv_ids, torch.from_numpy(send_eloc.astype(np.int64)), out_splits, in_splits)
        dist.all_to_all_single(recv_rows, torch.from_numpy(send_rows), out_splits, in_splits)
    rid = recv_ids.numpy()
    rr = recv_rows.numpy()
    out = np.zeros_like(rr)
    ok = rid != EMPTY_SLOT
    assert np.all(rid[ok] < epr)
    out[ok] = _fake_expert(rr[ok], (rid[ok] + rank * epr).astype(np.float32))
    back = torch.empty(slots, D)
    if fixed:
        dist.all_to_all_single(back, torch.from_numpy(out))
    else:
        dist.all_to_all_single(back, torch.from_numpy(out), in_splits, out_splits)
    back = back.numpy()
    y = np.zeros((T, D), dtype=np.float32)
    for t in range(T):
        for r in range(K):
            y[t] += w[t, r] * back[inverse[t * K + r]]
    ref = np.zeros((T, D), dtype=np.float32)
    for t in range(T):
        for r in range(K):
            e = np.float32(idx[t, r])
            ref[t] += w[t, r] * (x[t] * (1.0 + 0.125 * e) + e)
    np.save(os.path.join(out_dir, f"err_{rank}.npy"), np.array([np.abs(y - ref).max(), send_counts.sum()]))
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("world,fixed", [(2, True), (2, False), (4, False)])
def test_dispatch_combine_round_trip_gloo(tmp_path, world, fixed):
    T, K, E, D = 9, 4, 16, 24
    port = _free_port()
    mp.spawn(_worker, args=(world, port, fixed, T, K, E, D, str(tmp_path)), nprocs=world, join=True)
    for r in range(world):
        err, sent = np.load(tmp_path / f"err_{r}.npy")
        assert err < 1e-4 and sent == T * K


def test_plan_dispatch_orders_and_inverse():
    from turbo_fieldfare_b200.ep import EMPTY_SLOT, plan_dispatch
    idx = np.array([[5, 0, 3], [3, 7, 1], [0, 6, 2]], dtype=np.uint32)      # 8 experts, 2 per rank, 4 ranks
    tok, eloc, inv, counts = plan_dispatch(idx, 2, 4)
    # sorted by (expert, token, rank): experts 0,0,1,2,3,3,5,6,7
    assert tok.tolist() == [0, 2, 1, 2, 0, 1, 0, 2, 1]
    assert eloc.tolist() == [0, 0, 1, 0, 1, 1, 1, 0, 1]
    assert counts.tolist() == [3, 3, 1, 2]
    assert inv.reshape(3, 3).tolist() == [[6, 0, 4], [5, 8, 2], [1, 7, 3]]
    tok2, eloc2, inv2, _ = plan_dispatch(idx, 2, 4, capacity=4)
    assert tok2.tolist() == [0, 2, 1, -1, 2, 0, 1, -1, 0, -1, -1, -1, 2, 1, -1, -1]
    assert eloc2[3] == EMPTY_SLOT and inv2.reshape(3, 3).tolist() == [[8, 0, 5], [6, 13, 2], [1, 12, 4]]
    with pytest.raises(ValueError):
        plan_dispatch(np.zeros((5, 1), dtype=np.uint32), 2, 4, capacity=4)


def _lpt_reference(counts, world):
    """Numpy restatement of the rule tf_ep_balanced_placement documents."""
    L, E = counts.shape
    per = E // world
    out = np.zeros((L, E), dtype=np.uint32)
    for l in range(L):
        order = sorted(range(E), key=lambda e: (-int(counts[l, e]), e))
        used, load = [0] * world, [0] * world
        for e in order:
            free = [r for r in range(world) if used[r] < per]
            best = min(free, key=lambda r: (load[r], r))
            out[l, best * per + used[best]] = e
            used[best] += 1
            load[best] += int(counts[l, e])
    return out


@pytest.mark.parametrize("world", [1, 2, 4, 8])
def test_balanced_placement_is_a_permutation_and_levels_the_shards(world):
    """Host-only entry of the library (no device work): per layer a permutation, equal to the documented greedy rule,
    and never worse balanced than contiguous shards."""
    from turbo_fieldfare_b200 import _capi
    from turbo_fieldfare_b200.ep import balanced_placement, shard_imbalance
    lib = _capi.load()
    rng = np.random.default_rng(7 + world)
    L, E = 5, 128
    counts = np.floor(rng.pareto(1.2, size=(L, E)) * 100).astype(np.uint64)
    counts[3] = 11                                   # all equal: identity
    counts[4, :] = 0
    counts[4, 5] = 1000                              # one expert takes everything
    placement = balanced_placement(lib, counts, world)
    assert placement.shape == (L, E) and placement.dtype == np.uint32
    for l in range(L):
        assert sorted(placement[l].tolist()) == list(range(E))
    assert np.array_equal(placement, _lpt_reference(counts, world))
    before = shard_imbalance(counts, None, world)
    after = shard_imbalance(counts, placement, world)
    assert np.all(after <= before + 1e-12)
    if world > 1:
        # heavy-tailed loads: the greedy rule lands within 4/3 of the larger of (mean, largest single expert)
        per_rank_mean = counts[:3].sum(axis=1) / world
        bound = np.maximum(per_rank_mean, counts[:3].max(axis=1)) * (4.0 / 3.0)
        placed = np.take_along_axis(counts, placement.astype(np.int64), axis=1)[:3].reshape(3, world, -1).sum(axis=2).max(axis=1)
        assert np.all(placed <= bound + 1)


def test_balanced_placement_rejects_bad_arguments():
    from turbo_fieldfare_b200 import _capi
    from turbo_fieldfare_b200.ep import balanced_placement
    lib = _capi.load()
    with pytest.raises(ValueError):
        balanced_placement(lib, np.ones((2, 10), np.uint64), 4)          # 10 experts do not divide over 4 ranks
    with pytest.raises(ValueError):
        balanced_placement(lib, np.ones(10, np.uint64), 2)               # not [layers, experts]
