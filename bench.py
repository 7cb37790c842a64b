#!/usr/bin/env python
"""Headline benchmark: KV-cache block xcopy on the pooled HBM (device -> remote device), N GPUs of one node.

One step = one batched put of BLOCKS KV blocks (one block = 61 layers x (128 KiB K/V + 16 KiB rope) =
122 discrete segments, 8784 KiB) from a private device buffer into the NEXT rank's slice of the pool
(rank r -> (r + 1) % N; with one GPU the target is the rank's own slice), through the public API
``BigMemory.copy_data_batch`` = the C call ``smem_bm_copy_batch``: every step hands the library the 7808
(source, destination, size) triples again, so the validation of every triple, the merging of neighbours,
the cutting into work chunks and the writing of the descriptor ring are inside the timed region. The
value is the whole-job aggregate GB/s (10^9 B/s). Device-timed with CUDA events on the launching stream,
max over ranks. The per-step input (549 MiB) is larger than L2.

    python bench.py --gpus 1 --steps 20 --warmup 5
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 --master-port P \
        bench.py --gpus 8 --steps 20 --warmup 5
    python bench.py --impl reference ...      # the reference arm (prints an "unavailable" line, see below)
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

PUBLISHED_D2RD_GBS = 138.01  # reference README.md:128-129, xcopy D2RD 1 GB on Ascend A3


def host_pool_cfg1(impl: str) -> dict:
    """The CPU-only configuration both implementations can run: 2 processes, 64 MiB of pooled DRAM each, copy_data of
    4 KiB - 8 MiB to and from the peer's slice with CRC32 (baseline/host_pool_cfg1.py, its own process: it must import
    only ONE of the two ``memfabric_hybrid`` packages)."""
    import subprocess
    try:
        p = subprocess.run([sys.executable, os.path.join(ROOT, "baseline", "host_pool_cfg1.py"), "--impl", impl, "--iters", "1024"],
                           capture_output=True, text=True, timeout=600, cwd=os.path.join(ROOT, "baseline"))
        line = [l for l in p.stdout.splitlines() if l.startswith("{")]
        return json.loads(line[-1]) if line else {"impl": impl, "unavailable": (p.stderr or "no output")[-300:]}
    except Exception as e:  # noqa: BLE001
        return {"impl": impl, "unavailable": repr(e)[:300]}


def reference_arm(args) -> int:
    # Headline metric (device -> remote-device copies on pooled HBM): the reference ships no installable package at its
    # root (pip: "Neither 'setup.py' nor 'pyproject.toml' found"), its -DXPU_TYPE=GPU build does not compile unmodified
    # (dl_cuda_api.cpp: 'FileUtil' has not been declared), and on every non-NPU build smem_bm_create rejects all device
    # data paths, so that metric has no reference implementation to run. What the unmodified reference DOES run on this
    # box is its CPU-only flavour (-DXPU_TYPE=NONE, built into baseline/_ref): the host DRAM pool configuration is
    # measured through its own Python API and printed under "extras" for a same-box comparison.
    rank = int(os.environ.get("RANK", "0"))
    if rank == 0:
        print(json.dumps({"impl": "reference", "unavailable":
                          "reference is not pip-installable (no setup.py/pyproject.toml at its root); its XPU_TYPE=GPU build "
                          "fails to compile unmodified and non-NPU builds reject every device data path",
                          "extras": {"host_pool_cfg1": host_pool_cfg1("reference")}}))
    return 0


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--blocks", type=int, default=64, help="KV blocks per step")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--extras", type=int, default=1, help="also measure collectives / MoE when available")
    args = ap.parse_args()
    if args.impl == "reference":
        return reference_arm(args)
    if args.warmup < 3:
        args.warmup = 3

    import torch
    import torch.distributed as dist

    from memfabric_hybrid_b200.utils import benchutil as bu
    rank, world, local = bu.env_rank_world()
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torch.distributed.run")
    torch.cuda.set_device(local)
    # host staging buffers next to this rank's GPU: one process per GPU, each on the CPUs and memory of its GPU's NUMA node
    from memfabric_hybrid_b200.utils import numa
    numa_info = numa.bind_to_gpu(local) if os.environ.get("MF_NUMA_BIND", "1") != "0" else {"node": None}
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))

    import memfabric_hybrid as mf
    from memfabric_hybrid import bm

    mf.initialize()
    mf.set_log_level(int(os.environ.get("MF_LOG_LEVEL", "2")))
    cfg = bm.BmConfig()
    cfg.rank_id = rank
    cfg.start_store = rank == 0
    addr = os.environ.get("MASTER_ADDR", "127.0.0.1")
    port = int(os.environ.get("MASTER_PORT", "29500")) + 23
    if world == 1:
        import socket
        s = socket.socket()
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
        s.close()
    url = f"tcp://{addr}:{port}"
    rc = bm.initialize(url, world, local, cfg)
    assert rc == 0, f"bm.initialize: {rc} {mf.get_last_err_msg()}"

    nblk = args.blocks
    step_bytes = nblk * bu.KV_BLOCK_BYTES
    # the extras put up to 1024 KV blocks (8.6 GiB) and one 2 GiB run into the slice
    want_bytes = max(step_bytes, (1024 * bu.KV_BLOCK_BYTES) if args.extras else 0)
    pool_bytes = ((want_bytes + (64 << 20)) + (2 << 20) - 1) // (2 << 20) * (2 << 20)
    h = bm.create2(id=0, local_dram_size=0, max_dram_size=0, local_hbm_size=pool_bytes, max_hbm_size=pool_bytes,
                   data_op_type=bm.BmDataOpType.SDMA)
    assert h.join() == 0, mf.get_last_err_msg()
    bu.barrier()
    # join is dynamic: wait until every rank is a member and mapped here
    if world > 1:
        deadline = time.time() + 120
        while True:
            probe = torch.zeros(8, dtype=torch.uint8, device="cuda")
            ok = all(h.copy_data(h.peer_rank_ptr(r, bm.BmMemType.DEVICE), probe.data_ptr(), 8, bm.BmCopyType.G2L, 0) == 0
                     for r in range(world))
            if ok:
                break
            mf.get_and_clear_last_err_msg()
            assert time.time() < deadline, "peers did not join in time"
            time.sleep(0.05)
        bu.barrier()

    peer = (rank + 1) % world
    dst_base = h.peer_rank_ptr(peer, bm.BmMemType.DEVICE)
    src = torch.randn(step_bytes // 2, dtype=torch.bfloat16, device="cuda", generator=torch.Generator("cuda").manual_seed(rank))
    import numpy as np
    segs = bu.kv_block_segments(nblk)
    # the descriptor lists as a serving engine keeps them: arrays of 64-bit addresses and sizes
    srcs = np.array([src.data_ptr() + off for off, _ in segs], dtype=np.uint64)
    dsts = np.array([dst_base + off for off, _ in segs], dtype=np.uint64)
    sizes = np.array([sz for _, sz in segs], dtype=np.uint64)
    n = len(segs)
    stream = torch.cuda.Stream()
    flags = bm.ASYNC_COPY_FLAG | bm.FLAG_USE_EXTERNAL_STREAM

    def put():
        rc = h.copy_data_batch(srcs, dsts, sizes, n, bm.BmCopyType.L2G, flags, stream.cuda_stream)
        assert rc == 0, mf.get_last_err_msg()

    # ---- correctness of one put before timing: the peer's slice must equal the source bit for bit
    put()
    stream.synchronize()
    bu.barrier()
    check = torch.empty_like(src)
    prev = (rank - 1) % world
    me_base = h.peer_rank_ptr(rank, bm.BmMemType.DEVICE)
    assert h.copy_data(me_base, check.data_ptr(), step_bytes, bm.BmCopyType.G2L, 0) == 0, mf.get_last_err_msg()
    want = torch.randn(step_bytes // 2, dtype=torch.bfloat16, device="cuda", generator=torch.Generator("cuda").manual_seed(prev))
    assert torch.equal(check.view(torch.int16), want.view(torch.int16)), "KV blocks arrived corrupted"
    del check, want

    for _ in range(args.warmup):
        put()
    stream.synchronize()
    stats0 = h.copy_stats()
    sampler = bu.ClockSampler(local).start()
    bu.barrier()
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(2)]
    host_t0 = time.perf_counter()
    with torch.cuda.stream(stream):
        ev[0].record(stream)
        for _ in range(args.steps):
            put()
        ev[1].record(stream)
    host_us_per_call = (time.perf_counter() - host_t0) / args.steps * 1e6   # what the calling thread spends inside the API per step
    stream.synchronize()
    bu.barrier()
    clocks = sampler.stop()
    ms = bu.max_over_ranks(ev[0].elapsed_time(ev[1])) / args.steps
    stats1 = h.copy_stats()
    launches = stats1["kernel_launches"] - stats0["kernel_launches"]
    value = world * step_bytes / (ms * 1e-3) / 1e9

    # ---- end to end: pinned host -> device (H2D of the step's input), put, device -> host read of a result word
    host = torch.empty(step_bytes // 2, dtype=torch.bfloat16).pin_memory()
    host.copy_(src)
    result = torch.zeros(8, dtype=torch.uint8).pin_memory()
    tail = dst_base + step_bytes - 8

    def e2e_step():
        with torch.cuda.stream(stream):
            src.copy_(host, non_blocking=True)
        put()
        rc = h.copy_data(tail, result.data_ptr(), 8, bm.BmCopyType.G2H, flags, stream.cuda_stream)
        assert rc == 0, mf.get_last_err_msg()
        stream.synchronize()

    for _ in range(3):
        e2e_step()
    bu.barrier()
    t0 = time.perf_counter()
    e2e_steps = max(3, args.steps // 2)
    for _ in range(e2e_steps):
        e2e_step()
    torch.cuda.synchronize()
    e2e_ms = bu.max_over_ranks((time.perf_counter() - t0) * 1e3) / e2e_steps
    e2e_value = world * step_bytes / (e2e_ms * 1e-3) / 1e9
    bu.barrier()

    extras = {}
    if args.extras:
        try:
            from memfabric_hybrid_b200.utils import bench_extras
            extras = bench_extras.run(rank, world, local, h)
        except Exception as e:  # noqa: BLE001  (the headline number must not depend on the extras)
            extras = {"error": repr(e)[:200]}

    if rank == 0 and args.extras:
        extras["host_pool_cfg1"] = host_pool_cfg1("ours")
    if rank == 0:
        out = {
            "metric": "kv_block_xcopy_d2rd_GBps", "value": round(value, 2), "unit": "GB/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(ms, 4), "higher_is_better": True,
            "scaling": "weak", "vs_baseline": round(value / world / PUBLISHED_D2RD_GBS, 3), "dtype": "bf16", "data": "synthetic",
            "config": {"model": "DeepSeek-R1 KV block: 61 layers x (128 KiB + 16 KiB) = 122 segments, 8784 KiB",
                       "global_batch": world * nblk, "seq_len": bu.KV_SEGMENTS, "parallelism": f"ring-put x{world}",
                       "blocks_per_step": nblk, "bytes_per_step_per_gpu": step_bytes,
                       "l2": "inputs larger than L2 (549 MiB per step)",
                       "api": "memfabric_hybrid.bm.BigMemory.copy_data_batch = smem_bm_copy_batch (L2G, ASYNC_COPY_FLAG on a CUDA stream); "
                              "all 7808 triples are validated and marshalled by the library on every step",
                       "host_us_per_call": round(host_us_per_call, 1), "descriptors_per_call": n,
                       "per_gpu_GBps": round(value / world, 2), "numa": numa_info,
                       "vs_baseline_note": "per-GPU rate / 138.01 GB/s (reference D2RD, one 1 GB transfer on Ascend A3)",
                       "scaling_note": "with 1 GPU the 'remote' slice is the GPU's own HBM (no NVLink); from 2 GPUs on every put crosses "
                                       "NVLink, where stores issued by SMs reach 709 GB/s per direction between two B200s and copy engines 772"},
            "clocks": clocks,
            "e2e": {"value": round(e2e_value, 2), "unit": "GB/s", "h2d_bytes_per_step": step_bytes, "d2h_bytes_per_step": 8,
                    "ms_per_step": round(e2e_ms, 4)},
            "gpu_launches": int(launches),
            "extras": extras,
        }
        print(json.dumps(out))
    h.leave()
    bu.barrier()  # rank 0 hosts the config store: nobody tears down while a peer is still leaving
    h.destroy()
    bm.uninitialize(0)
    mf.uninitialize()
    if world > 1:
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
