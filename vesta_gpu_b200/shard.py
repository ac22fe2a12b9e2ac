"""Independent sequences partitioned over GPUs: one process per GPU, every rank holds the whole
model and runs the single-GPU step kernel on its own sequences. There is no exchange on the step
path; the generated token ids are gathered to rank 0 once at the end (torch.distributed: NCCL on
GPUs, gloo in CPU tests).

The reference is single-GPU (it has no distributed code); a batch there is "the same questions
asked of several tokens at once" (QUESTIONS.md:96), so sequences never interact and any split by
sequence is exact.
"""
import numpy as np


def partition(lengths, world):
    """Assign sequences to ranks, balancing the total context each rank reads: longest first,
    dealt to the least loaded rank. -> list (per rank) of sequence indices, ascending.

    lengths: per-sequence cost (e.g. prompt length + generated tokens); equal lengths give the
    contiguous split [r*B/G, (r+1)*B/G)."""
    lengths = np.asarray(lengths)
    B = len(lengths)
    if world < 1 or B % world:
        raise ValueError(f'{B} sequences do not split evenly over {world} ranks')
    per = B // world
    if np.all(lengths == lengths[0]):
        return [list(range(r * per, (r + 1) * per)) for r in range(world)]
    load = [0] * world
    out = [[] for _ in range(world)]
    for i in sorted(range(B), key=lambda i: (-int(lengths[i]), i)):
        r = min((r for r in range(world) if len(out[r]) < per), key=lambda r: (load[r], r))
        out[r].append(i)
        load[r] += int(lengths[i])
    return [sorted(v) for v in out]


def gather_tokens(local_tokens, mine, total, group=None, device=None):
    """Collect every rank's generated tokens on rank 0 in the original sequence order.

    local_tokens: int32 tensor [len(mine), steps] on this rank; mine: this rank's sequence indices
    (from partition); total: number of sequences over all ranks.
    -> on rank 0 an int32 tensor [total, steps]; None elsewhere."""
    import torch
    import torch.distributed as dist
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    if world == 1:
        out = torch.empty((total, local_tokens.shape[1]), dtype=local_tokens.dtype, device=local_tokens.device)
        out[torch.as_tensor(mine, device=local_tokens.device)] = local_tokens
        return out
    rank = dist.get_rank(group)
    steps = local_tokens.shape[1]
    idx = torch.as_tensor(mine, dtype=torch.int32, device=local_tokens.device)
    payload = torch.cat([idx[:, None], local_tokens.to(torch.int32)], dim=1).contiguous()
    # all_gather rather than gather: supported by every backend for device tensors, and 4 bytes per token
    bufs = [torch.empty_like(payload) for _ in range(world)]
    dist.all_gather(bufs, payload, group=group)
    if rank != 0:
        return None
    out = torch.empty((total, steps), dtype=torch.int32, device=local_tokens.device)
    for b in bufs:
        out[b[:, 0].long()] = b[:, 1:]
    return out
