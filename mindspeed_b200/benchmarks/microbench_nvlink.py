"""How fast can SMs write into peer memory over NVLink?  Guides the data-movement design of the fused GEMM + collective
kernels (csrc/kernels/gemm2_comm_sm100.cu).

  python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P \
      -m mindspeed_b200.benchmarks.microbench_nvlink [--mib 256]

Every rank pushes ``--mib`` MiB of a local buffer into its peers' symmetric buffers at once (all ranks send and receive
simultaneously, as in an all-gather).  Variants: bulk-copy (TMA) ring with 8 KB / 16 KB chunks and 4 / 8 slots, TMA stores
alone, plain 16-byte stores; destination = one peer, or chunks spread over all peers.  CUDA events around one launch after a
barrier, best of 5, minimum over ranks of GB/s per direction per GPU; NCCL all-gather of the same bytes for comparison.
"""
from __future__ import annotations

import argparse
import ctypes
import os

import torch
import torch.distributed as dist


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--mib", type=int, default=256)
    a = ap.parse_args()
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    from ..ops import gemm as G
    from ..ops import loader
    from ..parallel.symm_mem import destroy_heaps, get_heap
    L = loader.require_lib()
    nbytes = a.mib << 20
    heap = get_heap(dist.group.WORLD, nbytes + (1 << 20), tag="probe")
    off = heap.alloc("probe", nbytes)
    src = torch.randint(0, 255, (nbytes,), dtype=torch.uint8, device="cuda")
    peers = (ctypes.c_void_p * 8)(*[heap.ptr(r, off) for r in range(world)] + [None] * (8 - world))
    st = G.status_word(src.device)

    def run(mode, chunk, spread, ring, ctas=0):
        best = 1e9
        for _ in range(5):
            torch.cuda.synchronize()
            dist.barrier()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            loader.check(L.msb_nvlink_probe(ctypes.c_void_p(src.data_ptr()), peers, ctypes.c_size_t(nbytes), chunk, world, rank,
                                            spread, mode, ring, ctas, ctypes.c_void_p(st.data_ptr()),
                                            ctypes.c_void_p(loader.stream_ptr())), "nvlink_probe")
            e1.record()
            torch.cuda.synchronize()
            best = min(best, e0.elapsed_time(e1))
        G.check_status()
        t = torch.tensor([nbytes / best / 1e6], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MIN)
        return float(t.item())

    rows = []
    for spread in ((0, 1) if world > 2 else (0,)):
        for name, mode, chunk, ring in (("tma ring 8K x4", 0, 8192, 4), ("tma ring 8K x8", 0, 8192, 8), ("tma ring 16K x8", 0, 16384, 8),
                                        ("tma ring 16K x4", 0, 16384, 4), ("tma store only 16K", 2, 16384, 8), ("tma store only 4K", 2, 4096, 8),
                                        ("ld/st 16B", 1, 16384, 2)):
            rows.append((name, "all peers" if spread else "one peer", run(mode, chunk, spread, ring)))
    rows.append(("tma ring 16K x8, 32 CTAs", "all peers" if world > 2 else "one peer", run(0, 16384, 1 if world > 2 else 0, 8, 32)))
    # NCCL all-gather moving the same number of bytes out of every GPU
    per = nbytes // max(world - 1, 1)
    x = torch.empty(per, dtype=torch.uint8, device="cuda")
    out = torch.empty(per * world, dtype=torch.uint8, device="cuda")
    best = 1e9
    for _ in range(5):
        torch.cuda.synchronize(); dist.barrier(); torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(); dist.all_gather_into_tensor(out, x); e1.record(); torch.cuda.synchronize()
        best = min(best, e0.elapsed_time(e1))
    rows.append(("NCCL all_gather", "-", per * (world - 1) / best / 1e6))
    if rank == 0:
        print(f"# {world} GPUs, {a.mib} MiB pushed per GPU; GB/s per direction per GPU (minimum over ranks)")
        for name, pol, gbs in rows:
            print(f"{name:26s} {pol:10s} {gbs:8.1f} GB/s", flush=True)
    dist.barrier()
    destroy_heaps()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
