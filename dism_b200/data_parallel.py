"""Gradient sum of data-parallel replicas: the one collective of the path.

The hard operator itself needs none (every (batch, head) is independent); a model trained on several
GPUs keeps one replica per rank and adds the replicas' gradients once per step.  The reference does this
without a DDP wrapper: flat buckets of at most 16 MiB per (device, dtype), one all_reduce(SUM) each, after
an all_reduce(MAX) of a mask that tells which parameters got a gradient on any rank
(nanochat/nanochat/document_loss.py:13-53).  Same scheme here, over NCCL on NVLink for CUDA tensors and
over gloo in the CPU tests.
"""
import torch
import torch.distributed as dist


def bucket_plan(sizes, limit):
    """Greedy split of a list of byte sizes into consecutive buckets of at most `limit` bytes (a single larger
    entry gets a bucket of its own).  Returns a list of (first, end) index ranges."""
    plan, first, filled = [], 0, 0
    for index, size in enumerate(sizes):
        if index > first and filled + size > limit:
            plan.append((first, index))
            first, filled = index, 0
        filled += size
    if first < len(sizes):
        plan.append((first, len(sizes)))
    return plan


@torch.no_grad()
def sum_gradients(parameters, bucket_bytes=16 << 20, group=None):
    """Every rank leaves with the sum over ranks of each parameter's gradient.  A parameter without a gradient
    on this rank but with one elsewhere contributes zeros; one without a gradient on every rank keeps None."""
    parameters = list(parameters)
    if not parameters:
        return
    used = torch.tensor([p.grad is not None for p in parameters], device=parameters[0].device, dtype=torch.int32)
    dist.all_reduce(used, op=dist.ReduceOp.MAX, group=group)
    families = {}
    for parameter, flag in zip(parameters, used.tolist()):
        if not flag:
            continue
        if parameter.grad is None:
            parameter.grad = torch.zeros_like(parameter)
        if parameter.grad.is_sparse:
            raise ValueError('dense gradients required')
        families.setdefault((parameter.grad.device, parameter.grad.dtype), []).append(parameter.grad)
    for gradients in families.values():
        for first, end in bucket_plan([g.numel() * g.element_size() for g in gradients], bucket_bytes):
            members = gradients[first:end]
            flat = torch.cat([g.reshape(-1) for g in members])
            dist.all_reduce(flat, op=dist.ReduceOp.SUM, group=group)
            torch._foreach_copy_(members, [piece.view_as(g) for piece, g in zip(flat.split([g.numel() for g in members]), members)])
