"""Sharding a population over the GPUs of one box: one process per GPU, members split in
contiguous slices, no communication in the forward pass, one all-reduce of the concatenated
update per step (and one all-gather of fitness values when the fitness shaping is global).

The reference is single-GPU and has no counterpart; this is the data-parallel split its
member-independent forward (``modules/base.py:355-381,487-508``) and member-summed update
(``modules/base.py:110-138``) admit.  Works on any ``torch.distributed`` backend: NCCL over
NVLink on GPUs, gloo on CPU for tests of the host logic.
"""
import torch
import torch.distributed as dist


def member_slice(directions, rank, world_size):
    """Contiguous slice [lo, hi) of the member index owned by ``rank``; sizes differ by at most one."""
    if world_size <= 0 or not (0 <= rank < world_size):
        raise ValueError("bad rank/world_size")
    base, extra = divmod(directions, world_size)
    lo = rank * base + min(rank, extra)
    return lo, lo + base + (1 if rank < extra else 0)


def local_rows(batch, directions, rank, world_size):
    """Rows of a global batch (layout ``b = r * directions + d``) that belong to ``rank``'s
    members, as a (R, local_D, ...) -> (R * local_D, ...) re-batched tensor with the same layout
    for ``local_D`` directions."""
    lo, hi = member_slice(directions, rank, world_size)
    R = batch.shape[0] // directions
    return batch.view(R, directions, *batch.shape[1:])[:, lo:hi].reshape(R * (hi - lo), *batch.shape[1:])


def gather_fitness(local_fitness, group=None, sizes=None):
    """All ranks' per-member fitness, concatenated in rank order (ranks may own unequal slices).

    ``sizes`` (members per rank, in rank order) avoids the exchange of the slice sizes and, with it, the
    host synchronisation that reading them back costs: pass it whenever the split is known, e.g.
    ``[hi - lo for lo, hi in (member_slice(population, r, world) for r in range(world))]``."""
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size(group) == 1:
        return local_fitness
    world = dist.get_world_size(group)
    if sizes is None:
        counts = [torch.zeros(1, dtype=torch.int64, device=local_fitness.device) for _ in range(world)]
        dist.all_gather(counts, torch.tensor([local_fitness.numel()], dtype=torch.int64, device=local_fitness.device),
                        group=group)
        sizes = [int(c.item()) for c in counts]
    else:
        sizes = [int(n) for n in sizes]
        if len(sizes) != world or sizes[dist.get_rank(group)] != local_fitness.numel():
            raise ValueError("sizes must list every rank's member count, this rank's included")
    n_max = max(sizes)
    flat = local_fitness.flatten()
    if flat.numel() == n_max:
        padded = flat.contiguous()
    else:
        padded = torch.zeros(n_max, dtype=local_fitness.dtype, device=local_fitness.device)
        padded[:flat.numel()] = flat
    parts = [torch.empty_like(padded) for _ in range(world)]
    dist.all_gather(parts, padded, group=group)
    return torch.cat([p[:n] for p, n in zip(parts, sizes)])


class UpdateBucket:
    """One flat fp32 buffer that holds every partial gradient of a step, so that a step costs a
    single all-reduce whatever the number of layers."""

    def __init__(self, tensors):
        self.shapes = [tuple(t.shape) for t in tensors]
        self.sizes = [t.numel() for t in tensors]
        ref = tensors[0]
        self.flat = torch.empty(sum(self.sizes), dtype=torch.float32, device=ref.device)

    def views(self):
        out, off = [], 0
        for shape, n in zip(self.shapes, self.sizes):
            out.append(self.flat[off:off + n].view(shape))
            off += n
        return out

    def pack(self, tensors):
        for v, t in zip(self.views(), tensors):
            if v.data_ptr() != t.data_ptr():
                v.copy_(t)

    def attach(self, params):
        """Tell the layers to write the next gradients straight into this bucket: every parameter gets its slice
        as ``_nes_grad_out``, which the update kernels take as their output while ``.grad`` is empty."""
        for p, v in zip(params, self.views()):
            p._nes_grad_out = v

    def holds(self, tensors):
        """True when every tensor IS its slice of the bucket (nothing to pack, nothing to copy back)."""
        return all(v.data_ptr() == t.data_ptr() and v.shape == t.shape for v, t in zip(self.views(), tensors))

    def all_reduce(self, group=None):
        if dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1:
            dist.all_reduce(self.flat, op=dist.ReduceOp.SUM, group=group)
        return self.views()


def overlapped_dense_update(layer, weights, bucket=None, group=None, blocks=4, l1=0, l2=0):
    """Update of a dense-noise layer (``PerturbedLinear`` / ``PerturbedConv2d``) with the all-reduce taken off the
    critical path: the weight gradient is formed in ``blocks`` column blocks written straight into the bucket, and
    the all-reduce of block k is issued asynchronously while block k + 1 streams its share of the noise; only the
    last block's reduction (and the small bias reduction) is exposed.  Leaves the full-population gradients in
    ``.grad`` (slices of the bucket) and returns the bucket."""
    params = [layer.weight] + ([layer.bias] if layer.bias is not None else [])
    if bucket is None or bucket.sizes != [p.numel() for p in params]:
        bucket = UpdateBucket([p.detach() for p in params])
        bucket.attach(params)
    views = bucket.views()
    flat = views[0].view(-1)
    n = flat.numel()
    multi = dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1
    step = -(-n // max(1, int(blocks)))
    step = (step + 1023) // 1024 * 1024            # whole 4 KiB pieces: the 128-bit path and aligned collectives
    pending = []
    for lo in range(0, n, step):
        hi = min(n, lo + step)
        layer.weight_grad_columns(weights, lo, hi, flat[lo:hi], l1, l2)
        if multi:
            pending.append(dist.all_reduce(flat[lo:hi], op=dist.ReduceOp.SUM, group=group, async_op=True))
    layer.weight.grad = views[0]
    if layer.bias is not None:
        layer.bias.grad = None
        layer._weighted_sum(layer.bias_noise, weights, None, 0, 0, None, views[1])
        layer.bias.grad = views[1]
        if multi:
            pending.append(dist.all_reduce(views[1], op=dist.ReduceOp.SUM, group=group, async_op=True))
    for work in pending:
        work.wait()
    return bucket


def all_reduce_grads(parameters, bucket=None, group=None):
    """Sum ``.grad`` of the given parameters over the ranks through one bucket; every rank ends
    with the full-population update and applies the same optimiser step.

    The first call builds the bucket and attaches its slices to the parameters; from then on an update that
    starts from ``.grad = None`` writes its gradients directly into the bucket, the all-reduce runs in place and
    ``.grad`` is the reduced slice -- no packing and no copy back.  Gradients that live elsewhere (an accumulating
    update, a layer without the hook) are packed first and ``.grad`` is pointed at the reduced slice."""
    params = [p for p in parameters if p.grad is not None]
    if not params:
        return bucket
    grads = [p.grad for p in params]
    if bucket is None or bucket.sizes != [g.numel() for g in grads]:
        bucket = UpdateBucket(grads)
        bucket.attach(params)
    in_place = bucket.holds(grads)
    if not in_place:
        bucket.pack(grads)
    views = bucket.all_reduce(group)
    if not in_place:
        for p, v in zip(params, views):
            p.grad = v
    return bucket
