"""A reinforcement-learning weight hand-over: the actor is trained with tensor parallel 2 x pipeline parallel 2 (four
ranks, Megatron-style fused shards, experts spread over the ranks of a stage) and served by an inference engine with
tensor parallel 2 on ranks 1 and 3. Every parameter moves shard to shard through a tensor_rtl executor and arrives under
its inference name; nothing is ever gathered on one rank. The flow of the reference's examples/verl preprocessor.

    python examples/tensor_rtl/rl_train_to_infer_reshard.py
"""
import os
import sys

import torch

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), ".."))
import _launch  # noqa: E402

MODEL = dict(num_layers=4, hidden=64, ffn=96, heads=8, kv_heads=4, head_dim=8, vocab=200)


def build_full_blocks(specs, seed=7):
    """The whole model, block by block, identical on every rank (stands in for the trained weights)."""
    g = torch.Generator().manual_seed(seed)
    full = {}
    for s in specs:
        blocks = []
        for b in s.the_blocks():
            shape = list(s.shape)
            if s.shard_dim >= 0:
                shape[s.shard_dim] = b.size
            blocks.append(torch.randn(shape, generator=g))
        full[s.train_name] = blocks
    return full


def main(rank: int, world: int, port: int, moe: bool) -> str:
    import torch.distributed as dist
    from memfabric_hybrid_b200.tensor_rtl import All2AllVExecutor
    from memfabric_hybrid_b200.tensor_rtl.rl_reshard import (InferLayout, TrainLayout, TrainToInferResharder, decoder_specs,
                                                              train_shard_of)
    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
    cfg = dict(MODEL, num_experts=4, moe_ffn=32) if moe else MODEL
    specs, meta = decoder_specs(**cfg, fuse_for_inference=moe, qkv_bias=not moe, qk_norm=moe)   # dense: Qwen2-like, routed: Qwen3-like
    train = TrainLayout(tp=2, pp=2, ep=2 if moe else 1)
    infer = InferLayout(tp=2, ranks=[1, 3], ep=2 if moe else 1)
    job = TrainToInferResharder(specs, train, infer, rank, All2AllVExecutor(), meta, backend="gloo", bucket_bytes=64 << 10)
    full = build_full_blocks(specs)
    # what this rank holds while training
    state = {}
    for s in specs:
        mesh = job.train_mesh(s)
        if rank in mesh:
            state[s.train_name] = train_shard_of(s, full[s.train_name], len(mesh), mesh.index(rank))
    got = dict(job.per_tensor(state, dtype=torch.float32))
    # what the inference engine must have received
    ok, count = True, 0
    for s in specs:
        blocks = s.the_blocks()
        exp = [job.expected_infer_shard(s, i, full[s.train_name][i], rank) for i in range(len(blocks))]
        if exp[0] is None:
            ok &= all(b.infer_name not in got for b in blocks)
            continue
        if s.infer_fused_name and len(blocks) > 1:
            ok &= torch.equal(got[s.infer_fused_name], torch.cat(exp, dim=s.shard_dim))
            count += 1
        else:
            for b, e in zip(blocks, exp):
                ok &= torch.equal(got[b.infer_name], e)
                count += 1
    ok &= count == len(got)
    dist.barrier()
    dist.destroy_process_group()
    return f"ok {count} tensors, {job.moved_bytes >> 10} KiB moved" if ok else "mismatch"


if __name__ == "__main__":
    bad = 0
    for moe in (False, True):
        res = _launch.run(main, 4, _launch.free_port(), moe)
        print("moe" if moe else "dense", res)
        bad += not all(r.startswith("ok") for r in res)
    sys.exit(1 if bad else 0)
