"""Mesh arithmetic (pure) and the gradient reducer over gloo ranks."""
import torch

from conftest import free_port
from mp_util import run_ranks


def test_mesh_groups_partition_the_world():
    from memfabric_hybrid_b200.parallel import Mesh
    tp, dp, pp = 2, 2, 2
    world = tp * dp * pp
    for kind, size in (("tp", tp), ("dp", dp), ("pp", pp), ("ep", 4)):
        groups = {tuple(Mesh.ranks_of(kind, r, tp, dp, pp, 4)) for r in range(world)}
        assert all(len(g) == size for g in groups)
        assert sorted(r for g in groups for r in g) == list(range(world))            # a partition
        for g in groups:                                                             # evenly spaced: native zbal communicators
            steps = {g[i + 1] - g[i] for i in range(len(g) - 1)}
            assert len(steps) <= 1
    assert Mesh.ranks_of("tp", 5, tp, dp, pp, 4) == [4, 5]
    assert Mesh.ranks_of("dp", 5, tp, dp, pp, 4) == [5, 7]
    assert Mesh.ranks_of("pp", 5, tp, dp, pp, 4) == [1, 5]


def _reduce(rank, world, port):
    import torch.distributed as dist
    from memfabric_hybrid_b200.parallel import GradReducer, Mesh
    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
    mesh = Mesh(tp=2, pp=1)
    assert mesh.dp == 2 and mesh.tp_ranks == [rank // 2 * 2, rank // 2 * 2 + 1] and mesh.dp_ranks == [rank % 2, rank % 2 + 2]
    torch.manual_seed(0)
    model = torch.nn.Sequential(torch.nn.Linear(8, 16), torch.nn.Linear(16, 4))
    for i, p in enumerate(model.parameters()):
        p.grad = torch.full_like(p, float(rank + i))
    r = GradReducer(model.parameters(), group=mesh.dp_group, bucket_mb=1, symmetric=False)
    r.reduce()
    r.wait()
    for i, p in enumerate(model.parameters()):
        exp = sum(float(m + i) for m in mesh.dp_ranks) / 2
        assert torch.allclose(p.grad, torch.full_like(p, exp))
    dist.barrier()
    dist.destroy_process_group()
    return True


def test_grad_reducer_over_gloo():
    assert run_ranks(_reduce, 4, (free_port(),), timeout=120) == [True] * 4
