"""Resharding plans (pure functions) and the three executors on CPU: gloo ranks for the process-group
executors, a host-DRAM BigMemory pool for the memory-fabric executor."""
import os

import pytest
import torch

from conftest import free_port
from mp_util import run_ranks


def test_overlaps_cover_everything_once():
    from memfabric_hybrid_b200.tensor_rtl import overlaps, shard_bounds
    for size, old, new in ((4096, [0, 1, 2, 3], [4, 5]), (10, [0, 1, 2], [0, 1, 2, 3]), (7, [3], [0, 1, 2]), (12, [0, 1], [1, 0])):
        pieces = overlaps(size, old, new)
        cover = sorted((lo, hi) for _, _, lo, hi in pieces)
        assert cover[0][0] == 0 and cover[-1][1] == size
        assert all(cover[i][1] == cover[i + 1][0] for i in range(len(cover) - 1))
        for src, dst, lo, hi in pieces:
            a = shard_bounds(size, len(old), old.index(src))
            b = shard_bounds(size, len(new), new.index(dst))
            assert a[0] <= lo < hi <= a[1] and b[0] <= lo < hi <= b[1]


def test_validation_and_pack_roundtrip():
    from memfabric_hybrid_b200.tensor_rtl import PTensor, pack_tensors, unpack_tensors
    t = torch.zeros(4, 6)
    with pytest.raises(ValueError):
        PTensor(t, torch.float32, 2, [0, 1], (8, 6), 0, rank=0, backend="smoke signals")
    with pytest.raises(ValueError):
        PTensor(t, torch.float32, 2, [0, 0], (8, 6), 0, rank=0)
    with pytest.raises(ValueError):
        PTensor(t, torch.float32, 2, [0, 1], (12, 6), 0, rank=0)   # rank 0 would hold 6 rows, not 4
    ts = [torch.arange(7, dtype=torch.int32), torch.randn(3, 5).to(torch.bfloat16), torch.tensor([1.5], dtype=torch.float64)]
    packed, meta = pack_tensors(ts, torch.int32)
    assert packed.dtype == torch.int32
    back = unpack_tensors(packed, meta)
    assert all(torch.equal(a, b) and a.dtype == b.dtype for a, b in zip(ts, back))


def _global(shape, seed):
    return torch.arange(int(torch.tensor(shape).prod()), dtype=torch.float32).reshape(shape) + seed * 1000


def _reshard(rank, world, port, kind):
    import torch.distributed as dist
    from memfabric_hybrid_b200.tensor_rtl import (All2AllVExcutor, BatchP2PExecutor, MemoryFabricExecutor, MfBmConfig, PTensor, PTensorSet)
    os.environ["MF_DEVICE_BACKEND"] = "none"
    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
    # three tensors: rows TP4 (ranks 0-3) -> TP2 (ranks 2, 3); columns TP2 (0, 1) -> TP4 (all, uneven 10 columns); replicated -> rank 3
    specs = [((8, 6), 0, [0, 1, 2, 3], [2, 3]), ((4, 10), 1, [0, 1], [0, 1, 2, 3]), ((5,), -1, [0, 1], [3])]
    backend = "mf" if kind == "mf" else "gloo"
    pts = []
    for i, (shape, dim, old, new) in enumerate(specs):
        full = _global(shape, i)
        shard = None
        if rank in old:
            shard = full if dim < 0 else full.chunk(len(old), dim)[old.index(rank)].contiguous()
        pts.append(PTensor(shard, torch.float32, len(shape), old, shape, dim, rank=rank, backend=backend))
    ps = PTensorSet(pts)
    ps.transfer_map([s[3] for s in specs])
    if kind == "p2p":
        ex = BatchP2PExecutor()
    elif kind == "a2a":
        ex = All2AllVExcutor()
    else:
        ex = MemoryFabricExecutor(MfBmConfig(url=f"tcp://127.0.0.1:{port + 1}", local_dram_size=8 << 20, rank_world_size=world), rank_id=rank)
    ex.execute(ps.get_transfer_list())
    ex.wait()
    got = ps.collect_tensor()
    for i, (shape, dim, old, new) in enumerate(specs):
        full = _global(shape, i)
        if rank in new:
            if dim < 0:
                exp = full
            else:
                n, j = len(new), new.index(rank)
                lo, hi = shape[dim] * j // n, shape[dim] * (j + 1) // n
                exp = full.narrow(dim, lo, hi - lo)
            assert got[i] is not None and torch.equal(got[i], exp), f"tensor {i} on rank {rank}: {got[i]} vs {exp}"
        else:
            assert got[i] is None
    dist.barrier()
    if kind == "mf":
        MemoryFabricExecutor.shutdown()
    dist.destroy_process_group()
    return True


@pytest.mark.parametrize("kind", ["p2p", "a2a", "mf"])
def test_reshard_executors(kind):
    assert run_ranks(_reshard, 4, (free_port(), kind), timeout=180) == [True] * 4


def _reshard_twice(rank, world, port):
    import torch.distributed as dist
    from memfabric_hybrid_b200.tensor_rtl import BatchP2PExecutor, BufferPool, PTensor
    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
    # columns TP2 (ranks 0, 1) -> TP4 (all ranks): the senders' column slices are not contiguous, rank 0 and 1 keep a part
    shape, old, new = (4, 8), [0, 1], [0, 1, 2, 3]
    shard = torch.zeros(4, 4) if rank in old else None
    pt = PTensor(shard, torch.float32, 2, old, shape, 1, rank=rank, backend="gloo", reuse_buffers=True)
    assert isinstance(pt.buffer_pool, BufferPool)
    ptrs, ex = [], BatchP2PExecutor()
    for step in range(3):
        full = _global(shape, step)
        if rank in old:
            shard.copy_(full.chunk(2, 1)[old.index(rank)])       # the weights changed in place, as after an optimizer step
        pt.transfer_map(new)                                       # the same plan again
        ex.execute(pt.get_transfer_list())
        ex.wait()
        got = pt.collect_tensor()
        assert torch.equal(got, full.narrow(1, 2 * rank, 2)), (rank, step, got)
        ptrs.append((got.data_ptr(), tuple(sorted(b.data_ptr() for d in pt.buffer_pool.send_buffer_dict.values() for b in d.values()))))
        dist.barrier()
    assert ptrs[0] == ptrs[1] == ptrs[2]                            # nothing was allocated after the first round
    assert list(pt.buffer_pool.get_keys()) == [(2, 4)] and pt.buffer_pool.nbytes() > 0
    n_ops = len(pt.get_transfer_list())
    pt.transfer_map(new)
    assert len(pt.get_transfer_list()) == n_ops                     # a new plan replaces the old one instead of growing it
    dist.destroy_process_group()
    return True


def test_repeating_plan_reuses_its_buffers():
    assert run_ranks(_reshard_twice, 4, (free_port(),), timeout=120) == [True] * 4


def test_buffer_pool_and_small_helpers():
    from memfabric_hybrid_b200.tensor_rtl import (BaseCommTask, BatchP2PExecutor, BufferPool, Executor, MFCommTask, P2PCommTask, Planner,
                                                  get_dtype_size)
    import tensor_rtl
    assert tensor_rtl.BufferPool is BufferPool and tensor_rtl.get_dtype_size is get_dtype_size
    bp = BufferPool()
    a, b = torch.zeros(3), torch.ones(3)
    assert bp.get((2, 4), (0, 3)) is None
    bp.register((2, 4), (0, 3), a)
    bp.register((2, 4), (0, 3), b)                                 # the first registration wins
    assert bp.get((2, 4), (0, 3)) is a and list(bp.get_keys()) == [(2, 4)]
    assert bp.get_or_create((2, 4), (3, 6), lambda: b) is b and bp.get_or_create((2, 4), (3, 6), lambda: a) is b
    assert bp.nbytes() == 24
    bp.clear()
    assert bp.get((2, 4), (0, 3)) is None
    assert [get_dtype_size(d) for d in (torch.bool, torch.int8, torch.float8_e4m3fn, torch.bfloat16, torch.float32, torch.int64,
                                        torch.complex64)] == [1, 1, 1, 2, 4, 8, 8]
    assert issubclass(P2PCommTask, BaseCommTask) and issubclass(MFCommTask, BaseCommTask) and issubclass(BatchP2PExecutor, Executor)
    assert BatchP2PExecutor().batch_comm_list == []
    with pytest.raises(TypeError):
        Executor()                                                  # abstract

    class Reverse(Planner):
        def build_ordered_comm_ops(self, op_list):
            return list(reversed(op_list))
    t = [P2PCommTask(idx=i) for i in range(3)]
    assert [x.idx for x in Reverse(topology="ring").build_ordered_comm_ops(t)] == [2, 1, 0] and Planner().build_ordered_comm_ops(t) == t


def test_eplb_slot_pairing():
    from memfabric_hybrid_b200.tensor_rtl import pair_slots
    old = [0, 1, 2, 3, 0, 1]
    # nothing moves / a swap inside one rank / a replica pulled from the copy on its own rank / round-robin over holders
    assert pair_slots(old, old, 2) == []
    assert pair_slots([0, 1, 2, 3], [1, 0, 2, 3], 2) == [(1, 0), (0, 1)]
    assert pair_slots(old, [0, 0, 2, 3, 0, 1], 2) == [(0, 1)]
    assert pair_slots(old, [0, 1, 0, 0, 0, 1], 2) == [(0, 2), (4, 3)]
    with pytest.raises(KeyError):
        pair_slots(old, [9, 1, 2, 3, 0, 1], 2)
    with pytest.raises(ValueError):
        pair_slots(old, old[:-1], 2)


def test_rl_reshard_splits_fused_training_shards():
    """The block splitter of the train -> inference resharder: a Megatron linear_qkv shard (q, k, v interleaved per query
    group) and a linear_fc1 shard (gate, up) come apart into the separately sharded blocks, on every tensor-parallel rank."""
    from memfabric_hybrid_b200.tensor_rtl.rl_reshard import (InferLayout, TrainLayout, TrainToInferResharder, decoder_specs,
                                                              train_shard_of)
    specs, meta = decoder_specs(num_layers=2, hidden=32, ffn=48, heads=8, kv_heads=4, head_dim=4, vocab=64, qkv_bias=True, qk_norm=True)
    qkv = next(s for s in specs if s.train_name.endswith("layers.0.self_attention.linear_qkv.weight"))
    bias = next(s for s in specs if s.train_name.endswith("layers.0.self_attention.linear_qkv.bias"))
    fc1 = next(s for s in specs if s.train_name.endswith("layers.1.mlp.linear_fc1.weight"))
    norms = [s for s in specs if "layernorm.weight" in s.train_name and ("q_layernorm" in s.train_name or "k_layernorm" in s.train_name)]
    assert len(norms) == 4 and all(s.shard_dim == -1 and s.shape == (4,) for s in norms)
    assert [b.infer_name.rsplit(".", 2)[-2:] for b in bias.the_blocks()] == [["q_proj", "bias"], ["k_proj", "bias"], ["v_proj", "bias"]]
    g = torch.Generator().manual_seed(1)
    for spec in (qkv, fc1, bias):
        full = [torch.randn(*((b.size, 32) if len(spec.shape) == 2 else (b.size,)), generator=g) for b in spec.the_blocks()]
        for tp in (1, 2, 4):
            for t in range(tp):
                job = TrainToInferResharder(specs, TrainLayout(tp=tp, pp=1), InferLayout(tp=1, ranks=[0]), rank=t, executor=None, meta=meta)
                local = train_shard_of(spec, full, tp, t)
                assert local.shape[0] == sum(b.size for b in spec.the_blocks()) // tp
                parts = job._local_blocks(spec, local, list(range(tp)))
                for blk, whole in zip(parts, full):
                    n = whole.shape[0] // tp
                    assert torch.equal(blk, whole[t * n:(t + 1) * n])
    # stages and expert placement
    tl = TrainLayout(tp=4, pp=2, ep=2)
    assert tl.stage_ranks(1) == [4, 5, 6, 7] and tl.stage_of_layer(3, 8) == 0 and tl.stage_of_layer(4, 8) == 1
    assert tl.expert_ranks(1, 5, 8) == [6, 7] and InferLayout(tp=2, ranks=[3, 9], ep=2).expert_ranks(5, 8) == [9]
    with pytest.raises(ValueError):
        TrainLayout(tp=4, pp=1, ep=3)


def test_eplb_planner_evens_out_a_skewed_router():
    """balanced_placement + remap_topk: a Zipf-like router that sends 2.4 x the mean to one rank ends within 10 % of the mean
    once the hottest experts have copies on spare slots; every token still reaches a copy of the expert it chose."""
    from memfabric_hybrid_b200.tensor_rtl import balanced_placement, remap_topk, replica_table
    world, local, spare, K, T = 8, 28, 4, 8, 4096
    E = world * local
    g = torch.Generator().manual_seed(0)
    logits = torch.randn(T, E, generator=g) - 0.4 * torch.log(torch.arange(1, E + 1, dtype=torch.float32))[None, :]
    idx = torch.topk(torch.softmax(logits, -1), K, dim=-1).indices.to(torch.int32)
    idx[3, 2] = -1
    load = torch.bincount(idx[idx >= 0].long(), minlength=E).float()
    before = load.view(world, local).sum(1)
    assert float(before.max() / before.mean()) > 1.8
    placement = balanced_placement(load.tolist(), world, local + spare)
    assert len(placement) == world * (local + spare) and set(placement) == set(range(E))
    table, counts = replica_table(placement, E)
    assert int(counts.sum()) == len(placement) and int(counts.max()) > 1
    phys = remap_topk(idx, table, counts)
    assert phys[3, 2] == -1 and phys.shape == idx.shape
    # every physical slot a token was sent to holds the logical expert the router chose
    pl = torch.tensor(placement)
    sel = phys >= 0
    assert torch.equal(pl[phys[sel].long()], idx[sel].long())
    after = torch.bincount(phys[sel].long() // (local + spare), minlength=world).float()
    assert float(after.max() / after.mean()) < 1.10, after
    # no rank holds two copies of one expert while another rank could have taken it
    for r in range(world):
        held = placement[r * (local + spare):(r + 1) * (local + spare)]
        assert len(set(held)) == len(held)
    with pytest.raises(ValueError):
        balanced_placement([1.0] * 10, 2, 4)


def test_eplb_planner_keeps_weights_in_place_when_it_can():
    """With the placement in force as a hint, a small change of the load moves few experts, a large one still rebalances,
    and the balance is not worse than the tolerance allows."""
    import random
    from memfabric_hybrid_b200.tensor_rtl import balanced_placement, pair_slots
    ep, per, E = 8, 8, 56
    rng = random.Random(3)
    load = [100.0 / (1 + e) ** 0.6 for e in range(E)]
    rng.shuffle(load)
    base = balanced_placement(load, ep, per)
    assert balanced_placement(load, ep, per, previous=base) == base              # nothing changed: nothing moves

    def imbalance(pl, ld):
        cp = [pl.count(e) for e in range(E)]
        w = [0.0] * ep
        for s, e in enumerate(pl):
            w[s // per] += ld[e] / cp[e]
        return max(w) / (sum(w) / ep)
    drift = [v * rng.uniform(0.9, 1.1) for v in load]                            # the router drifts a little
    cold, warm = balanced_placement(drift, ep, per), balanced_placement(drift, ep, per, previous=base)
    moved_cold, moved_warm = len(pair_slots(base, cold, per)), len(pair_slots(base, warm, per))
    assert moved_warm < moved_cold // 2, (moved_warm, moved_cold)
    assert imbalance(warm, drift) < imbalance(cold, drift) + 0.06 and imbalance(warm, drift) < 1.15
    assert sorted(warm) == sorted(cold)                                           # the same copies, placed differently
    hot = list(load)
    hot[7] *= 12                                                                  # one expert becomes very hot
    moved = balanced_placement(hot, ep, per, previous=base)
    assert moved.count(7) > base.count(7) and imbalance(moved, hot) < imbalance(base, hot) - 0.3
    with pytest.raises(ValueError):
        balanced_placement(load, ep, per, previous=base[:-1])
