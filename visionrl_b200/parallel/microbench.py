"""Timing of the fused collective kernels against their NCCL formulations.

    torchrun --nproc-per-node N --master-addr 127.0.0.1 -m visionrl_b200.parallel.microbench [--only NAME]

Every number is CUDA-event time on the launching stream after warm-up, the MAXIMUM over ranks, with
a buffer larger than the L2 written between iterations.  Rank 0 prints one JSON line per case:

* ``gather_gemm``      F1: ``x @ W.T`` with W row-sharded — one fused kernel (peer loads inside the
                       GEMM) against ``all_gather_into_tensor`` + the plain GEMM.  Bytes over NVLink per
                       rank = ``(N-1)/N`` of the weight; roofline = max(FLOPs / measured GEMM peak,
                       bytes / link bandwidth).
* ``bucket_reduce``    F2: reduce-scatter ⊕ cast ⊕ scale ⊕ fp32 accumulate of one block's gradients
                       against ``reduce_scatter_tensor`` + ``add_``.  Each rank reads ``(N-1)/N`` of
                       its slice from peers.
* ``weight_broadcast`` F4: one table-driven kernel storing this rank's shards into every replica,
                       then the version flag, against ``all_gather_into_tensor``.  Each rank sends
                       ``(N-1)`` copies of its shard.
* ``ulysses_layer``    F3: QKV-prepare with peer stores + attention with peer-store epilogue against
                       QKV-prepare + three ``all_to_all_single`` + attention + one ``all_to_all_single``.
* ``barrier``          the bounded flag barrier against ``dist.barrier``-style NCCL all-reduce of one
                       element.
"""

from __future__ import annotations

import argparse
import json
import os
import sys

import torch
import torch.distributed as dist

LINK_GBS = 770.0          # measured peer-copy bandwidth per direction per GPU on this hardware (nominal 900)
GEMM_TFLOPS = 1388.0      # measured sustained cuBLAS bf16 throughput


def _time(fn, iters: int, warmup: int, flush: torch.Tensor | None) -> float:
    for _ in range(warmup):
        fn()
    dist.barrier()
    torch.cuda.synchronize()
    total = 0.0
    for _ in range(iters):
        if flush is not None:
            flush.add_(1)
        dist.barrier()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        torch.cuda.synchronize()
        total += a.elapsed_time(b)
    t = torch.tensor([total / iters], device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def main(argv=None) -> int:
    parser = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    parser.add_argument("--only", default=None)
    parser.add_argument("--iters", type=int, default=10)
    parser.add_argument("--warmup", type=int, default=3)
    args = parser.parse_args(argv)

    from visionrl_b200.ops import _ext
    from visionrl_b200.parallel.mesh import ProcessMesh, init_distributed
    from visionrl_b200.parallel.symm import SymmetricPool

    rank, world, local = init_distributed()
    if world < 2:
        print(json.dumps({"error": "needs at least two ranks (torchrun)"}))
        return 1
    dev = torch.device("cuda", local)
    mesh = ProcessMesh.build()
    pool = SymmetricPool(mesh)
    ext = _ext.load()
    flush = torch.zeros(96 << 20, device=dev, dtype=torch.float32)        # 384 MB > L2
    out = []

    def report(row: dict) -> None:
        row.update(n_gpus=world)
        out.append(row)
        if rank == 0:
            print(json.dumps(row), flush=True)

    def want(name: str) -> bool:
        return args.only in (None, name)

    # ---------------------------------------------------------------------------- F1
    if want("gather_gemm"):
        for (m, n, k) in [(18848, 4608, 1536), (18848, 6144, 1536), (18848, 1536, 6144), (16, 9216, 1536)]:
            if n % world:
                continue
            rows = n // world
            shard = pool.allocate(rows * k, torch.bfloat16, dev, "w").view(rows, k)
            shard.copy_(torch.randn(rows, k, device=dev) * 0.02)
            full = torch.empty(n, k, device=dev, dtype=torch.bfloat16)
            ready = torch.zeros(16, device=dev, dtype=torch.int32)
            x = torch.randn(m, k, device=dev, dtype=torch.bfloat16)
            peers = pool.peer_pointers(shard.view(-1))
            torch.cuda.synchronize()
            pool.barrier()

            def fused():
                return ext.gemm_allgather(x, peers, full, ready, None, 0, rank, world, None, None, 0, False)[0]

            def library():
                dist.all_gather_into_tensor(full.view(-1), shard.reshape(-1))
                return ext.gemm_bf16(x, full, None, None, None, 0, 0, False, False, False)

            def gemm_only():
                return ext.gemm_bf16(x, full, None, None, None, 0, 0, False, False, False)

            ref = library()
            got = fused()
            err = (got.float() - ref.float()).abs().max().item()
            t_f, t_l, t_g = (_time(f, args.iters, args.warmup, flush) for f in (fused, library, gemm_only))
            flops = 2.0 * m * n * k
            link_bytes = (world - 1) / world * n * k * 2
            bound_ms = max(flops / (GEMM_TFLOPS * 1e9), link_bytes / (LINK_GBS * 1e6))
            report({"case": "gather_gemm", "m": m, "n": n, "k": k, "fused_ms": round(t_f, 4),
                    "nccl_plus_gemm_ms": round(t_l, 4), "gemm_alone_ms": round(t_g, 4),
                    "nvlink_gb": round(link_bytes / 1e9, 4),
                    "nvlink_gbs_if_exposed": round(link_bytes / 1e6 / t_f, 1),
                    "roofline_ms": round(bound_ms, 4), "frac_of_roofline": round(bound_ms / t_f, 3),
                    "max_abs_diff_vs_library": round(err, 5)})
            pool.barrier()

    # ---------------------------------------------------------------------------- F2
    if want("bucket_reduce"):
        elems = 84_934_656 // (8 * world) * (8 * world)       # one SD3.5-M block's weights
        stage = pool.allocate(elems, torch.bfloat16, dev, "stage")
        stage.copy_(torch.randn(elems, device=dev) * 0.01)
        shard_n = elems // world
        gshard = torch.zeros(shard_n, device=dev, dtype=torch.float32)
        table = torch.tensor([[rank * shard_n, 0, shard_n]], dtype=torch.int64, device=dev)
        peers = pool.peer_pointers(stage)
        part = torch.empty(shard_n, device=dev, dtype=torch.bfloat16)
        torch.cuda.synchronize()
        pool.barrier()

        def fused():
            ext.bucket_reduce_acc(peers, table, gshard, 1.0 / world, world, rank, shard_n)

        def library():
            dist.reduce_scatter_tensor(part, stage, op=dist.ReduceOp.SUM)
            gshard.add_(part.float(), alpha=1.0 / world)

        gshard.zero_()
        fused()
        a = gshard.clone()
        gshard.zero_()
        library()
        err = (a - gshard).abs().max().item()
        t_f, t_l = (_time(f, args.iters, args.warmup, flush) for f in (fused, library))
        link_bytes = (world - 1) * shard_n * 2                 # peers' copies of my slice
        report({"case": "bucket_reduce", "elements": elems, "fused_ms": round(t_f, 4),
                "nccl_plus_add_ms": round(t_l, 4), "nvlink_gb_in": round(link_bytes / 1e9, 4),
                "nvlink_gbs": round(link_bytes / 1e6 / t_f, 1),
                "frac_of_link": round(link_bytes / 1e6 / t_f / LINK_GBS, 3),
                "max_abs_diff_vs_library": round(err, 6)})
        pool.barrier()

    # ---------------------------------------------------------------------------- F4
    if want("weight_broadcast"):
        total = 2_007_760_896 // 2 // (8 * world) * (8 * world)    # half of the SD3.5-M block weights (bounded memory)
        shard_n = total // world
        shards = pool.allocate(shard_n, torch.bfloat16, dev, "shards")
        shards.copy_(torch.randn(shard_n, device=dev) * 0.02)
        replica = pool.allocate(total, torch.bfloat16, dev, "replica")
        table = torch.tensor([[0, rank * shard_n, shard_n]], dtype=torch.int64, device=dev)
        slot = pool.reserve_slots(16)
        version = [0]
        torch.cuda.synchronize()
        pool.barrier()

        def fused():
            version[0] += 1
            ext.p2p_broadcast_table(shards, pool.peer_pointers(replica), table, world, rank, shard_n)
            pool.signal(slot + rank, version[0])
            pool.wait(slot, world, version[0])

        def library():
            dist.all_gather_into_tensor(replica, shards)

        fused()
        a = replica.clone()
        library()
        same = bool(torch.equal(a, replica))
        t_f, t_l = (_time(f, args.iters, args.warmup, flush) for f in (fused, library))
        link_bytes = (world - 1) * shard_n * 2
        report({"case": "weight_broadcast", "elements": total, "fused_ms": round(t_f, 4),
                "nccl_all_gather_ms": round(t_l, 4), "nvlink_gb_out": round(link_bytes / 1e9, 4),
                "nvlink_gbs": round(link_bytes / 1e6 / t_f, 1),
                "frac_of_link": round(link_bytes / 1e6 / t_f / LINK_GBS, 3), "equal_to_library": same})
        pool.check("weight_broadcast")
        pool.barrier()

    # ---------------------------------------------------------------------------- F3
    if want("ulysses_layer"):
        from visionrl_b200.ops.attention import attention
        from visionrl_b200.ops.qkv import qkv_prepare
        from visionrl_b200.parallel.ulysses import SequenceParallel, _all_to_all_heads, _all_to_all_seq

        mesh_sp = ProcessMesh(rank=rank, world_size=world, dp=1, sp=world, sp_group=dist.group.WORLD)
        sp = SequenceParallel(mesh_sp, pool)
        heads, dh = next(h for h in (12, 40, 16, 32) if h % world == 0), 128    # Wan-1.3B / Wan-14B head counts first
        s_full = 14040 // (8 * world) * (8 * world)
        s_loc, b = s_full // world, 2
        qkv = torch.randn(b, s_loc, 3 * heads * dh, device=dev, dtype=torch.bfloat16)
        qw = torch.ones(heads * dh, device=dev, dtype=torch.bfloat16)
        kw = torch.ones(heads * dh, device=dev, dtype=torch.bfloat16)
        ang = torch.rand(s_loc, dh // 2, device=dev) * 6.28
        rope = (torch.cos(ang), torch.sin(ang))

        def fused():
            with torch.no_grad():
                return sp.fused_attention(qkv, heads, qw, kw, rope)

        def library():
            with torch.no_grad():
                q, k, v = qkv_prepare(qkv, heads, qw, kw, rope=rope)
                qh, kh, vh = (_all_to_all_heads(t.contiguous(), dist.group.WORLD, world) for t in (q, k, v))
                o = attention(qh, kh, vh)
                return _all_to_all_seq(o.contiguous(), dist.group.WORLD, world).transpose(1, 2).reshape(b, s_loc, -1)

        got, ref = fused().clone(), library()
        err = (got.float() - ref.float()).abs().max().item()
        t_f, t_l = (_time(f, args.iters, args.warmup, flush) for f in (fused, library))
        link_bytes = (world - 1) / world * 4 * b * s_loc * heads * dh * 2       # q, k, v out + o out
        report({"case": "ulysses_layer", "batch": b, "seq": s_full, "heads": heads, "head_dim": dh,
                "fused_ms": round(t_f, 4), "nccl_all_to_all_ms": round(t_l, 4),
                "nvlink_gb_out": round(link_bytes / 1e9, 4), "max_abs_diff_vs_library": round(err, 5)})
        pool.check("ulysses_layer")
        pool.barrier()

    # ---------------------------------------------------------------------------- barrier
    if want("barrier"):
        one = torch.zeros(1, device=dev)
        t_f = _time(pool.barrier, args.iters * 5, args.warmup, None)
        t_l = _time(lambda: dist.all_reduce(one), args.iters * 5, args.warmup, None)
        report({"case": "barrier", "flag_barrier_ms": round(t_f, 4), "nccl_allreduce_1elem_ms": round(t_l, 4)})
        pool.check("barrier")

    dist.barrier()
    dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    sys.exit(main())
