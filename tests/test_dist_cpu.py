"""Host logic of the member sharding, on CPU with world_size 2 over gloo."""
import os
import socket
import sys

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from conftest import ROOT


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank, world, port, out):
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from nesgpu_b200 import dist as nd
    from oracle import perturbed_ref as O
    D, R, n_in, n_out = 7, 2, 5, 4          # 7 members over 2 ranks: slices of 4 and 3
    g = torch.Generator().manual_seed(0)     # same tensors on every rank
    x = torch.randn(R * D, n_in, generator=g)
    W = torch.randn(n_out, n_in, generator=g)
    E = torch.randn(D, n_out, n_in, generator=g)
    beta = torch.randn(D, n_out, generator=g)
    fitness = torch.randn(D, generator=g)
    lo, hi = nd.member_slice(D, rank, world)
    xl = nd.local_rows(x, D, rank, world)
    # forward of the local slice needs no communication and equals the rows of the global forward
    yl = O.perturbed_linear_forward(xl, W, None, E[lo:hi], beta[lo:hi], hi - lo, True)
    yg = O.perturbed_linear_forward(x, W, None, E, beta, D, True)
    ok = torch.allclose(yl, nd.local_rows(yg, D, rank, world), atol=1e-6)
    # fitness gathered in rank order with unequal slice sizes
    allfit = nd.gather_fitness(fitness[lo:hi].clone())
    ok &= torch.equal(allfit, fitness)
    # the same with the split given (no size exchange); a wrong split is refused
    known = [h - l for l, h in (nd.member_slice(D, r, world) for r in range(world))]
    ok &= torch.equal(nd.gather_fitness(fitness[lo:hi].clone(), sizes=known), fitness)
    try:
        nd.gather_fitness(fitness[lo:hi].clone(), sizes=[D, D])
        ok = False
    except ValueError:
        pass
    # partial updates summed through one bucket
    wgt = O.centered_ranks(allfit)
    wpar = torch.nn.Parameter(W.clone())
    bpar = torch.nn.Parameter(torch.zeros(n_out))
    wpar.grad, bpar.grad = O.perturbed_update(W, E[lo:hi], beta[lo:hi], wgt[lo:hi])
    bucket = nd.all_reduce_grads([wpar, bpar])
    full_w, full_b = O.perturbed_update(W, E, beta, wgt)
    ok &= torch.allclose(wpar.grad, full_w, atol=1e-5) and torch.allclose(bpar.grad, full_b, atol=1e-5)
    ok &= bucket.flat.numel() == n_out * n_in + n_out
    # the bucket is reused on the next step
    wpar.grad, bpar.grad = O.perturbed_update(W, E[lo:hi], beta[lo:hi], 2 * wgt[lo:hi])
    ok &= nd.all_reduce_grads([wpar, bpar], bucket) is bucket
    ok &= torch.allclose(wpar.grad, 2 * full_w, atol=1e-5)
    # the first call attached the bucket's slices to the parameters: an update that writes there is reduced in place
    ok &= wpar._nes_grad_out.data_ptr() == bucket.views()[0].data_ptr()
    part_w, part_b = O.perturbed_update(W, E[lo:hi], beta[lo:hi], wgt[lo:hi])
    wpar.grad = bpar.grad = None
    wpar._nes_grad_out.copy_(part_w)
    bpar._nes_grad_out.copy_(part_b)
    wpar.grad, bpar.grad = wpar._nes_grad_out, bpar._nes_grad_out
    ok &= bucket.holds([wpar.grad, bpar.grad])
    ok &= nd.all_reduce_grads([wpar, bpar], bucket) is bucket
    ok &= torch.allclose(wpar.grad, full_w, atol=1e-5) and wpar.grad.data_ptr() == bucket.views()[0].data_ptr()
    # every rank tells its layers where its member slice starts in the population
    from nesgpu_b200 import es

    class Recorder:
        offset = None

        def set_member_offset(self, first):
            self.offset = first
    rec = Recorder()
    ok &= es.assign_member_offsets(rec, D) == lo and rec.offset == lo
    firsts = [torch.zeros(1, dtype=torch.int64) for _ in range(world)]
    dist.all_gather(firsts, torch.tensor([rec.offset]))
    ok &= len({int(f) for f in firsts}) == world                  # distinct on every rank
    out[rank] = bool(ok)
    dist.barrier()
    dist.destroy_process_group()


def test_member_slice_partitions():
    from nesgpu_b200 import dist as nd
    for D in (1, 7, 8, 1024, 8192):
        for world in (1, 2, 3, 8):
            cuts = [nd.member_slice(D, r, world) for r in range(world)]
            assert cuts[0][0] == 0 and cuts[-1][1] == D
            assert all(a[1] == b[0] for a, b in zip(cuts, cuts[1:]))
            sizes = [hi - lo for lo, hi in cuts]
            assert max(sizes) - min(sizes) <= 1


def test_two_ranks_gloo():
    world = 2
    port = _free_port()
    with mp.Manager() as m:
        out = m.dict()
        mp.spawn(_worker, args=(world, port, out), nprocs=world, join=True)
        assert dict(out) == {0: True, 1: True}


def test_auto_chunk():
    from nesgpu_b200 import es
    assert es.auto_chunk(1024, 256) == 64 and es.auto_chunk(64, 256) == 256 and es.auto_chunk(8192, 256) == 8
    assert es.auto_chunk(100000, 256) == 1 and es.auto_chunk(1, 7) == 7 and es.auto_chunk(65536, 256) == 1
    # with the SM count the calls fill whole waves of 128-row tiles: 74 x 1024 rows = 592 tiles = 4 x 148
    assert es.auto_chunk(1024, 256, 148) == 74 and es.auto_chunk(64, 256, 148) == 256 and es.auto_chunk(8192, 256, 148) == 8
