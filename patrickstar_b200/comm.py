"""The chunk collectives of one communication group, on any backend.

A communication group is ``world`` consecutive chunks of the fp16 chunk list;
chunk ``k`` of the group belongs to rank ``k`` (patrickstar/core/chunk_list.py:383-387).
The group's chunks are stored contiguously, so both collectives run in place on
one flat buffer with no flatten copy (the reference uses the tensor-list API,
patrickstar/core/client.py:481-485, 831-836, which makes torch gather the list
into a temporary first).  Works on CUDA tensors over NCCL (the product path)
and on CPU tensors over gloo (host-logic tests).
"""
import torch.distributed as dist


def reduce_scatter_group(group_buf, rank, world_size, chunk_size, process_group=None, async_op=False):
    """client.py:831-836 — SUM reduce-scatter: afterwards slice ``rank`` of
    ``group_buf`` holds the sum over ranks of that slice.  The reference's
    following ``payload /= world_size`` (client.py:838) is NOT applied here; the
    step kernel folds it into its gradient load."""
    assert group_buf.numel() == world_size * chunk_size
    out = group_buf[rank * chunk_size:(rank + 1) * chunk_size]
    return dist.reduce_scatter_tensor(out, group_buf, op=dist.ReduceOp.SUM, group=process_group,
                                      async_op=async_op)


def all_gather_group(group_buf, rank, world_size, chunk_size, process_group=None, async_op=False):
    """client.py:481-485 — all-gather of the group's chunks from their owners."""
    assert group_buf.numel() == world_size * chunk_size
    mine = group_buf[rank * chunk_size:(rank + 1) * chunk_size]
    return dist.all_gather_into_tensor(group_buf, mine, group=process_group, async_op=async_op)


def all_reduce_flag(flag, process_group=None):
    """patrickstar/ops/fp16_cpu_adam.py:292-297 — MAX all-reduce of the overflow
    flag.  The result stays where the flag lives; nothing is read back."""
    return dist.all_reduce(flag, op=dist.ReduceOp.MAX, group=process_group)
