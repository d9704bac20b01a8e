"""Host-side plumbing for traces sharded by contiguous record range over several ranks.

Each rank owns whole CUPTI buffers and a contiguous range of CPU ops.  The event text of a record
depends on its own bytes, scalars, and the correlation join, so the only data that must cross ranks is
the join keys: every rank's EXTERNAL_CORRELATION records (16 bytes each, processing order) and CPU-op
ids (4 bytes each).  `gather_join_keys` all-gathers both in rank order, which is global processing
order, so "last writer wins" (libkineto/src/CuptiActivityProfiler.cpp:293-296) is decided by position
in the gathered array exactly as in a single-process run.  Works with any torch.distributed backend
(NCCL on GPUs, gloo on CPUs).
"""
from __future__ import annotations


def gather_join_keys(ext_local, ops_local, rank: int, world: int, dist):
    """ext_local: int64 tensor with 2 words per record; ops_local: int32 tensor.
    Returns (ext_all, ops_all, own_begin): the gathered arrays in rank order and the index of this
    rank's first EXTERNAL_CORRELATION record in ext_all."""
    import torch

    dev = ext_local.device
    counts = torch.tensor([ext_local.numel() // 2, ops_local.numel()], dtype=torch.int64, device=dev)
    all_counts = torch.empty(world * 2, dtype=torch.int64, device=dev)
    dist.all_gather_into_tensor(all_counts, counts)
    all_counts = all_counts.view(world, 2).cpu()
    max_ext, max_ops = int(all_counts[:, 0].max()), int(all_counts[:, 1].max())
    ext_pad = torch.zeros(max(1, max_ext) * 2, dtype=torch.int64, device=dev)
    ext_pad[:ext_local.numel()] = ext_local
    ops_pad = torch.zeros(max(1, max_ops), dtype=torch.int32, device=dev)
    ops_pad[:ops_local.numel()] = ops_local
    ext_g = torch.empty(world * ext_pad.numel(), dtype=torch.int64, device=dev)
    ops_g = torch.empty(world * ops_pad.numel(), dtype=torch.int32, device=dev)
    dist.all_gather_into_tensor(ext_g, ext_pad)
    dist.all_gather_into_tensor(ops_g, ops_pad)
    # drop the padding: rank order is processing order
    ext_all = torch.cat([ext_g[r * ext_pad.numel(): r * ext_pad.numel() + int(all_counts[r, 0]) * 2] for r in range(world)])
    ops_all = torch.cat([ops_g[r * ops_pad.numel(): r * ops_pad.numel() + int(all_counts[r, 1])] for r in range(world)])
    own_begin = int(all_counts[:rank, 0].sum())
    return ext_all, ops_all, own_begin


def output_bases(out_bytes: int, rank: int, world: int, dist, device):
    """All-gathers the per-shard text sizes; returns (this shard's byte offset in the whole file's
    activities section, total bytes).  CPU-op events of all shards precede GPU events in the
    reference's file; callers that need that exact order place the two parts separately."""
    import torch

    mine = torch.tensor([out_bytes], dtype=torch.int64, device=device)
    sizes = torch.empty(world, dtype=torch.int64, device=device)
    dist.all_gather_into_tensor(sizes, mine)
    sizes = sizes.cpu()
    return int(sizes[:rank].sum()), int(sizes.sum())
