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
    rank's first EXTERNAL_CORRELATION record in ext_all.  Two collectives: the counts, then one
    packed payload (records and ids in one buffer, padded to the largest shard)."""
    import torch

    dev = ext_local.device
    n_ext, n_ops = ext_local.numel() // 2, ops_local.numel()
    counts = torch.tensor([n_ext, n_ops], dtype=torch.int64, device=dev)
    all_counts = torch.empty(world * 2, dtype=torch.int64, device=dev)
    dist.all_gather_into_tensor(all_counts, counts)
    all_counts = all_counts.view(world, 2).tolist()
    max_ext = max(1, max(c[0] for c in all_counts))
    max_ops = max(1, max(c[1] for c in all_counts))
    ops_words = (max_ops + 1) // 2                       # op ids packed two per 64-bit word
    stride = max_ext * 2 + ops_words
    pack = torch.empty(stride, dtype=torch.int64, device=dev)
    pack[:n_ext * 2] = ext_local
    pack[max_ext * 2:].view(torch.int32)[:n_ops] = ops_local
    gathered = torch.empty(world * stride, dtype=torch.int64, device=dev)
    dist.all_gather_into_tensor(gathered, pack)
    g = gathered.view(world, stride)
    if all(c[0] == max_ext for c in all_counts):
        ext_all = g[:, :max_ext * 2].reshape(-1)
    else:
        ext_all = torch.cat([g[r, :all_counts[r][0] * 2] for r in range(world)])
    gi = g[:, max_ext * 2:].view(torch.int32)
    if all(c[1] == max_ops for c in all_counts) and max_ops % 2 == 0:
        ops_all = gi.reshape(-1)
    else:
        ops_all = torch.cat([gi[r, :all_counts[r][1]] for r in range(world)])
    own_begin = sum(c[0] for c in all_counts[:rank])
    return ext_all.contiguous(), ops_all.contiguous(), own_begin


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
