"""
Data-parallel step on real GPUs (one process per GPU, world size 2; skipped with fewer than two
GPUs): the library's own NVLink-multicast all-reduce against exact sums, and the all-reduced
``.grad`` of a step through the autograd function against the full-batch gradient computed with the
same kernels, for the NCCL transport and for the library's kernel.  The reference has no distributed
code; what is checked is the contract of the harness: SUM over row shards reproduces the full batch.

The children run with NCCL's own multicast (NVLS) switched off; no rank leaves early and nothing
here provokes a time-out.
"""

import os
import socket

import pytest
import torch

pytestmark = pytest.mark.gpu


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(('127.0.0.1', 0))
        return s.getsockname()[1]


def _init(rank, world_size, port):
    import torch.distributed as dist
    os.environ['MASTER_ADDR'] = '127.0.0.1'
    os.environ['MASTER_PORT'] = str(port)
    os.environ['NCCL_NVLS_ENABLE'] = '0'
    torch.cuda.set_device(rank)
    dist.init_process_group('nccl', rank=rank, world_size=world_size, device_id=torch.device('cuda', rank))
    return dist


def _all_reduce_worker(rank, world_size, port):
    dist = _init(rank, world_size, port)
    try:
        import attorch_b200
        from attorch_b200.dp import _MultimemBucket
        device = torch.device('cuda', rank)
        for dtype, numel in ((torch.bfloat16, 1 << 20), (torch.float32, 3 * 4096 + 4), (torch.float16, 8 * 1001)):
            bucket = _MultimemBucket(numel, dtype, device, None, ctas=4)
            gen = torch.Generator(device=device).manual_seed(7)
            parts = [(torch.randn(numel, device=device, generator=gen) * (r + 1)).to(dtype) for r in range(world_size)]
            expected = sum(p.float() for p in parts)
            for repeat in range(3):                      # the barriers count launches: call it repeatedly
                bucket.flat.copy_(parts[rank])
                torch.cuda.synchronize()
                dist.barrier()
                bucket.all_reduce(0, numel)
                torch.cuda.synchronize()
                attorch_b200.check_status()
                tol = 1e-6 if dtype is torch.float32 else 1e-2
                torch.testing.assert_close(bucket.flat.float(), expected, rtol=tol, atol=tol)
                # Every rank holds the same bits.
                mine = bucket.flat.clone()
                other = [torch.empty_like(mine) for _ in range(world_size)]
                dist.all_gather(other, mine)
                assert all(torch.equal(o, mine) for o in other)
            # A sub-range (16-byte aligned) leaves the rest alone.
            bucket.flat.fill_(1.0)
            torch.cuda.synchronize()
            dist.barrier()
            bucket.all_reduce(8, 8 + 64)
            torch.cuda.synchronize()
            assert torch.all(bucket.flat[8:72] == world_size) and torch.all(bucket.flat[:8] == 1) \
                and torch.all(bucket.flat[72:] == 1)
            dist.barrier()
            del bucket
    finally:
        dist.destroy_process_group()


def _step_worker(rank, world_size, port, transport, exchange_dtype):
    dist = _init(rank, world_size, port)
    try:
        import attorch_b200
        from attorch_b200.dp import GradientBuckets
        device = torch.device('cuda', rank)
        rows, k, n = 384, 512, 640
        torch.manual_seed(5)
        layers = [attorch_b200.Linear(k, n, act_func='gelu', device=device), attorch_b200.Linear(n, k, device=device)]
        full = [attorch_b200.Linear(k, n, act_func='gelu', device=device), attorch_b200.Linear(n, k, device=device)]
        for a, b in zip(layers, full):
            b.load_state_dict(a.state_dict())
        buckets = GradientBuckets(layers, overlap=True, dw_chunks=2, comm_sms=32, grad_dtype=exchange_dtype,
                                  transport=transport)
        assert buckets.transport == transport
        gen = torch.Generator(device=device).manual_seed(50 + rank)
        x = torch.randn(rows, k, device=device, generator=gen)
        dy = (torch.randn(rows, k, device=device, generator=gen) * 0.01).bfloat16()
        for _ in range(2):                               # twice: the second step overwrites the first
            buckets.zero_grad()
            xg = x.clone().requires_grad_(True)
            with torch.autocast('cuda', dtype=torch.bfloat16):
                y = layers[1](layers[0](xg))
            y.backward(dy)
            buckets.finish()
        xs = [torch.empty_like(x) for _ in range(world_size)]
        dys = [torch.empty_like(dy) for _ in range(world_size)]
        dist.all_gather(xs, x)
        dist.all_gather(dys, dy)
        xf = torch.cat(xs).requires_grad_(True)
        with torch.autocast('cuda', dtype=torch.bfloat16):
            yf = full[1](full[0](xf))
        yf.backward(torch.cat(dys))
        torch.cuda.synchronize()
        attorch_b200.check_status()
        for got_layer, want_layer in zip(layers, full):
            # What an optimizer reads is the bucket itself.
            assert got_layer.weight.grad.data_ptr() == (buckets.flat_grad if buckets.widen else buckets.flat)[
                buckets._offsets[layers.index(got_layer)]:].data_ptr()
            torch.testing.assert_close(got_layer.weight.grad, want_layer.weight.grad, rtol=1e-2, atol=1e-2)
            torch.testing.assert_close(got_layer.bias.grad, want_layer.bias.grad, rtol=1e-2, atol=1e-2)
        torch.testing.assert_close(xg.grad, xf.grad[rank * rows:(rank + 1) * rows], rtol=1e-2, atol=1e-2)
    finally:
        dist.destroy_process_group()


def test_collective_wait_runs_out_and_reports():
    """
    The bounded wait of the all-reduce kernel, on one GPU: launched as rank 0 of 2 with a flag block for
    "rank 1" that nothing ever signals, its first cross-rank barrier gives up after the 2 s limit, the
    kernel skips the data phase (no multicast address is ever touched) and returns; the status word then
    holds AB200_DEV_TIMEOUT_COLLECTIVE and the device keeps working.
    """
    import time
    from attorch_b200 import _lib
    lib = _lib.load()
    device = torch.device('cuda', 0)
    words = lib.ab200_collective_flag_bytes() // 4
    flags = [torch.zeros(words, dtype=torch.int32, device=device) for _ in range(2)]
    blocks = torch.tensor([f.data_ptr() for f in flags], dtype=torch.int64, device=device)
    data = torch.ones(4096, dtype=torch.bfloat16, device=device)     # stands in for the bucket; never accessed
    status = torch.zeros(1, dtype=torch.int32, device=device)
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    rc = lib.ab200_multimem_all_reduce(data.data_ptr(), data.numel(), _lib.BF16, 0, 2, blocks.data_ptr(), 2,
                                       status.data_ptr(), torch.cuda.current_stream().cuda_stream)
    assert rc == 0
    torch.cuda.synchronize()
    elapsed = time.perf_counter() - t0
    assert int(status.item()) == 4                                   # AB200_DEV_TIMEOUT_COLLECTIVE
    assert _lib.error_string(4).startswith('device: all-reduce gave up')
    assert 1.5 < elapsed < 10.0
    assert torch.all(data == 1)                                      # the data phase was skipped
    assert float((torch.ones(8, device=device) * 2).sum()) == 16.0   # the context is still usable


def _spawn(fn, *args):
    if torch.cuda.device_count() < 2:
        pytest.skip('needs two GPUs')
    import torch.multiprocessing as mp
    mp.spawn(fn, args=(2, _free_port()) + args, nprocs=2, join=True)


def test_multimem_all_reduce_sums_and_repeats():
    _spawn(_all_reduce_worker)


@pytest.mark.parametrize('transport,exchange_dtype', [('nccl', None), ('nccl', torch.bfloat16),
                                                      ('multimem', None), ('multimem', torch.bfloat16)])
def test_data_parallel_step_matches_full_batch(transport, exchange_dtype):
    _spawn(_step_worker, transport, exchange_dtype)
