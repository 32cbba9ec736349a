"""One evolution-strategies step over a population-batched model: the step sequence of the
reference's trainers (``mnisttest.py:127-157``: set_noise -> perturbed forward -> per-member loss ->
centring -> update), with the population sharded over ranks as in :mod:`nesgpu_b200.dist`.

Every member sees the same minibatch of ``R`` examples; the batch handed to the model is laid out
``b = r * directions + d`` (reference ``modules/base.py:357``).  The forward is run in chunks of
examples so that activation memory stays bounded for large populations.
"""
import torch
import torch.nn.functional as F

from . import dist as ndist


def centered_ranks(fitness):
    """rank / (n - 1) - 1/2 with a stable sort (ties keep member order)."""
    n = fitness.numel()
    order = torch.argsort(fitness, stable=True)
    ranks = torch.empty(n, dtype=torch.float32, device=fitness.device)
    ranks[order] = torch.arange(n, dtype=torch.float32, device=fitness.device)
    return ranks / max(n - 1, 1) - 0.5


def update_weights(fitness, noise_scale=None, lr_scale=1.0):
    """Per-member weights handed to ``update`` so that ``.grad`` is a DESCENT direction of the loss, as in the
    reference's trainer: there ``update`` receives ``(loss - loss.mean()) * lr_scale / noise_scale``
    (``mnisttest.py:136-146``), ``.grad`` estimates +grad(loss) and ``torch.optim.SGD.step()`` descends.

    Here the fitness is the NEGATIVE loss and is rank-normalised, so the weights are
    ``-centered_ranks(fitness) * lr_scale / noise_scale``: the members with the highest loss (lowest fitness)
    get the largest positive weights.  ``noise_scale=None`` leaves the division out."""
    w = -centered_ranks(fitness)
    scale = float(lr_scale) / float(noise_scale) if noise_scale else float(lr_scale)
    return w if scale == 1.0 else w * scale


def model_noise_scale(perturbed_model):
    """The noise scale the model's perturbed layers are set to (that of the first layer that has one)."""
    for layer in perturbed_model.perturbed_layers:
        if getattr(layer, "noise_scale", None):
            return layer.noise_scale
    return None


def assign_member_offsets(perturbed_model, population, group=None):
    """Tell every perturbed layer the global index of this rank's first member (``set_member_offset``), so that
    ranks which share seeds draw different members.  Returns that index."""
    on = torch.distributed.is_available() and torch.distributed.is_initialized()
    rank = torch.distributed.get_rank(group) if on else 0
    world = torch.distributed.get_world_size(group) if on else 1
    lo = ndist.member_slice(population, rank, world)[0]
    perturbed_model.set_member_offset(lo)
    return lo


def takes_shared_input(perturbed_model):
    """True when the model's first perturbed layer declares ``options["shared_input"]``: it then receives the
    minibatch itself instead of its copy per member."""
    for m in perturbed_model.model.modules():
        if hasattr(m, "perturbed_flag") and hasattr(m, "options"):
            return bool(m.options.get("shared_input"))
    return False


PAIRS_PER_CHUNK = 65536      # member-example pairs per forward call: launches amortised, activations bounded (a few GB)


def auto_chunk(directions, examples, sms=None):
    """Examples per forward call such that a call evaluates about ``PAIRS_PER_CHUNK`` member-example pairs
    (64 for 1024 members; the whole minibatch for small populations, where launches would dominate).

    With ``sms`` (the GPU's SM count) the size is adjusted by up to a quarter either way so that the calls fill whole
    waves: the layer kernels work through a call in tiles of 128 batch rows, one tile per SM at a time, and a call of
    64 x 1024 rows is 512 tiles = 3.46 waves of 148 SMs, while 74 x 1024 rows are exactly four.  Among the even sizes
    in range (antithetic layers halve every call) the one with the fewest waves over the whole minibatch wins; ties go
    to the size nearest the plain choice."""
    base = max(1, min(int(examples), PAIRS_PER_CHUNK // max(int(directions), 1)))
    if not sms or base >= int(examples) or base < 8:
        return base
    best, best_cost = base, None
    for c in range(max(2, (base * 3) // 4), (base * 5) // 4 + 1):
        if c % 2:
            continue
        cost, left = 0, int(examples)
        while left > 0:
            n = min(c, left)
            tiles = -(-n * int(directions) // 128)
            cost += -(-tiles // int(sms))
            left -= n
        if best_cost is None or cost < best_cost or (cost == best_cost and abs(c - base) < abs(best - base)):
            best, best_cost = c, cost
    return best


_side_streams = {}


def _streams(device, n):
    """The launching stream plus n - 1 side streams of the device (created once)."""
    main = torch.cuda.current_stream(device)
    key = (device.index if device.index is not None else torch.cuda.current_device(), n)
    if key not in _side_streams:
        _side_streams[key] = [torch.cuda.Stream(device=device) for _ in range(n - 1)]
    return [main] + _side_streams[key]


def population_fitness(perturbed_model, inputs, labels, directions, chunk=None, streams=1):
    """Negative mean cross-entropy of every member on the shared minibatch: (directions,) tensor.
    ``chunk`` = examples per forward call (default: :func:`auto_chunk`).  With antithetic layers every call is split
    into its own + half and - half (``modules/base.py:377-378`` applies the sign by position in the call's batch), so
    the chunk size then decides which examples meet which sign; pass ``chunk=len(inputs)`` for the reference's split.

    With ``streams`` > 1 successive calls alternate over that many CUDA streams (the launching one and side
    streams), so that kernels of neighbouring calls that do not compete for the same resource (a streaming pre-pass
    next to a tensor-core kernel) can overlap; everything is joined back into the launching stream before the result
    is returned.  Whether it pays depends on the kernels: on the small CNN two streams saved 0.28 ms of 6.1 ms in the
    bf16 mode and cost 0.9 ms in the TF32 mode, whose fp32 activations are four times larger."""
    R = inputs.shape[0]
    if chunk is None:
        # whole waves per call pay when the calls run one after another (measured on the small CNN: 7.90 -> 7.67 ms);
        # with several streams equal calls balance the streams better (5.39 -> 5.56 ms with the adjusted size)
        one_stream = inputs.is_cuda and int(streams) <= 1
        sms = torch.cuda.get_device_properties(inputs.device).multi_processor_count if one_stream else None
        chunk = auto_chunk(directions, R, sms)
    shared = takes_shared_input(perturbed_model)
    starts = list(range(0, R, chunk))
    lanes = _streams(inputs.device, max(1, min(int(streams), len(starts)))) if inputs.is_cuda else [None]
    main = lanes[0]
    partial = [torch.zeros(directions, device=inputs.device, dtype=torch.float32) for _ in lanes]
    for side in lanes[1:]:
        side.wait_stream(main)            # inputs, labels and the zeroed sums are ready
    with torch.no_grad():
        for i, r0 in enumerate(starts):
            lane = i % len(lanes)
            r1 = min(R, r0 + chunk)
            rc = r1 - r0
            with torch.cuda.stream(lanes[lane]) if lanes[lane] is not None else _Null():
                if shared:
                    xb = inputs[r0:r1].contiguous()
                else:
                    xb = inputs[r0:r1].unsqueeze(1).expand(rc, directions, *inputs.shape[1:]).reshape(
                        rc * directions, *inputs.shape[1:])
                logits = perturbed_model.forward(xb)
                target = labels[r0:r1].repeat_interleave(directions)
                ce = F.cross_entropy(logits.view(rc * directions, -1), target, reduction="none")
                partial[lane] += ce.view(rc, directions).sum(dim=0)
    loss_sum = partial[0]
    for side, part in zip(lanes[1:], partial[1:]):
        main.wait_stream(side)
        loss_sum = loss_sum + part
    return -(loss_sum / R)


class _Null:
    def __enter__(self):
        return self

    def __exit__(self, *exc):
        return False


def es_step(perturbed_model, inputs, labels, directions, noise_scale=None, chunk=None, bucket=None, group=None,
            new_noise=True, population=None, reseed=True, streams=1, lr_scale=1.0):
    """set_noise -> fitness of the local members -> global centred ranks -> local update -> one all-reduce.

    ``directions`` is the number of members owned by this rank; ``population`` (optional) the number of members
    over all ranks, split as :func:`nesgpu_b200.dist.member_slice` does.  Returns (local fitness, bucket); the
    full-population gradient is left in ``.grad`` of the model's parameters on every rank.  It is a descent
    gradient (see :func:`update_weights`): follow the step with an ordinary minimising optimiser
    (``torch.optim.SGD(...).step()``), as the reference's trainer does.

    With ``population`` given and more than one rank, every layer is told the global index of its first member
    (``set_member_offset``), so that ranks which share seeds still draw different members: the population is then
    ``population`` distinct members, not copies of one rank's slice.  Layers must share their seeds across ranks
    for the noise that all members share (``Permuted`` / ``Synthetic`` weight noise): seed Python's ``random``
    identically on all ranks, or pass ``reseed=False`` after setting the same seeds everywhere."""
    rank = torch.distributed.get_rank(group) if (torch.distributed.is_available() and torch.distributed.is_initialized()) else 0
    world = torch.distributed.get_world_size(group) if (torch.distributed.is_available() and torch.distributed.is_initialized()) else 1
    if population is not None:
        assign_member_offsets(perturbed_model, population, group)
    if new_noise:
        # noise is a pure function of each layer's seed, so a step draws new seeds first, as the reference's
        # trainer does (mnisttest.py:128-131); reseed=False keeps the seeds that are set
        if reseed:
            perturbed_model.set_seed()
        perturbed_model.set_noise(noise_scale)
    fitness = population_fitness(perturbed_model, inputs, labels, directions, chunk, streams)
    # with the population size given, every rank knows the split and the step needs no host synchronisation
    known = None if population is None else [hi - lo for lo, hi in (ndist.member_slice(population, r, world) for r in range(world))]
    everyone = ndist.gather_fitness(fitness, group, known)
    weights_all = update_weights(everyone, model_noise_scale(perturbed_model), lr_scale)
    # ranks own contiguous member slices in rank order (sizes may differ by one)
    sizes = [ndist.member_slice(everyone.numel(), r, world) for r in range(world)]
    lo, hi = sizes[rank]
    for p in perturbed_model.model.parameters():
        p.grad = None
    with torch.no_grad():
        perturbed_model.update(weights_all[lo:hi].contiguous())
    bucket = ndist.all_reduce_grads(perturbed_model.model.parameters(), bucket, group)
    return fitness, bucket
