"""
Data-parallel logic on CPU ranks (gloo, world size 2): row sharding, zero-copy gradient buckets and
the SUM all-reduce reproduce the single-process full-batch gradient.  The per-rank gradients come
from the CPU oracle, since the CUDA kernels need a GPU.
"""

import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import attorch_b200
from attorch_b200.dp import GradientBuckets, shard_rows
from oracle import linear_oracle as oracle


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(('127.0.0.1', 0))
        return s.getsockname()[1]


def _inputs():
    gen = torch.Generator().manual_seed(0)
    x = torch.randn(64, 24, generator=gen)
    w1 = torch.randn(24, 32, generator=gen) / 5
    b1 = torch.randn(32, generator=gen)
    w2 = torch.randn(32, 16, generator=gen) / 6
    b2 = torch.randn(16, generator=gen)
    dy = torch.randn(64, 16, generator=gen)
    return x, w1, b1, w2, b2, dy


def _two_layer_grads(x, w1, b1, w2, b2, dy):
    h, z1 = oracle.linear_forward(x, w1, b1, 'gelu')
    y, _ = oracle.linear_forward(h, w2, b2, None)
    dh, dw2, db2 = oracle.linear_backward(dy, h, None, w2, None, torch.float32, b2)
    _, dw1, db1 = oracle.linear_backward(dh, x, z1, w1, 'gelu', torch.float32, b1)
    return dw1, db1, dw2, db2


def _worker(rank: int, world_size: int, port: int, overlap_requested: bool, defer: bool = False) -> None:
    os.environ['MASTER_ADDR'] = '127.0.0.1'
    os.environ['MASTER_PORT'] = str(port)
    dist.init_process_group('gloo', rank=rank, world_size=world_size)
    try:
        x, w1, b1, w2, b2, dy = _inputs()
        layers = [attorch_b200.Linear(24, 32, act_func='gelu', device='cpu'),
                  attorch_b200.Linear(32, 16, device='cpu')]
        buckets = GradientBuckets(layers, overlap=overlap_requested, defer_first_input_grad=defer)
        assert buckets.world_size == world_size
        assert (layers[0].defer_input_grad is not None) == defer and layers[1].defer_input_grad is None
        assert not buckets.overlap            # side streams exist only on CUDA
        assert buckets.flat.numel() == 24 * 32 + 32 + 32 * 16 + 16       # already whole 16-byte units
        # The gradient destinations alias the flat bucket.
        assert layers[0].weight_grad_out.data_ptr() == buckets.flat.data_ptr()
        xs, dys = shard_rows(x, rank, world_size), shard_rows(dy, rank, world_size)
        dw1, db1, dw2, db2 = _two_layer_grads(xs, w1, b1, w2, b2, dys)
        layers[0].weight_grad_out.copy_(dw1)
        layers[0].bias_grad_out.copy_(db1)
        layers[1].weight_grad_out.copy_(dw2)
        layers[1].bias_grad_out.copy_(db2)
        for layer in layers:
            layer.grad_ready()
        launched = []
        if defer:
            # What backward would hand over instead of launching the first layer's dX.
            layers[0].defer_input_grad(lambda: launched.append(rank))
            buckets.start_exchange()          # CPU ranks: the exchange happens in finish()
            buckets.run_deferred()
            assert launched == [rank] and not buckets._deferred
        buckets.finish()
        f_dw1, f_db1, f_dw2, f_db2 = _two_layer_grads(x, w1, b1, w2, b2, dy)
        torch.testing.assert_close(layers[0].weight_grad_out, f_dw1, rtol=1e-5, atol=1e-5)
        torch.testing.assert_close(layers[0].bias_grad_out, f_db1, rtol=1e-5, atol=1e-5)
        torch.testing.assert_close(layers[1].weight_grad_out, f_dw2, rtol=1e-5, atol=1e-5)
        torch.testing.assert_close(layers[1].bias_grad_out, f_db2, rtol=1e-5, atol=1e-5)
        # What an optimizer reads: every .grad is the bucket itself, so it holds the sum over ranks.
        assert layers[0].weight.grad.data_ptr() == buckets.flat.data_ptr()
        torch.testing.assert_close(layers[0].weight.grad, f_dw1, rtol=1e-5, atol=1e-5)
        torch.testing.assert_close(layers[1].bias.grad, f_db2, rtol=1e-5, atol=1e-5)
        buckets.zero_grad()
        assert layers[1].weight.grad.data_ptr() == layers[1].weight_grad_out.data_ptr()
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize('overlap', [False, True])
def test_data_parallel_gradients_match_full_batch(overlap):
    mp.spawn(_worker, args=(2, _free_port(), overlap), nprocs=2, join=True)


def test_deferred_input_gradient_step():
    mp.spawn(_worker, args=(2, _free_port(), False, True), nprocs=2, join=True)


def test_shard_rows():
    t = torch.arange(24).view(8, 3)
    assert torch.equal(shard_rows(t, 1, 4), t[2:4])
    with pytest.raises(ValueError):
        shard_rows(t, 0, 3)


def test_single_process_bucket_is_a_no_op():
    layer = attorch_b200.Linear(4, 6, device='cpu')
    buckets = GradientBuckets([layer])
    layer.weight_grad_out.fill_(2.0)
    buckets.finish()
    assert torch.all(layer.weight_grad_out == 2.0)


def test_grads_alias_the_bucket():
    """
    ``.grad`` of every parameter is a view of the flat bucket from construction on (backward writes
    the bucket and returns no gradient of its own for these parameters, so autograd never replaces
    the alias with a copy), and ``zero_grad`` restores an alias that something dropped.
    """
    layers = [attorch_b200.Linear(4, 6, device='cpu'), attorch_b200.Linear(6, 2, bias=False, device='cpu')]
    buckets = GradientBuckets(layers)
    assert buckets.flat.numel() == 44          # 4 * 6 + 6 + 6 * 2 = 42 fp32, padded to whole 16-byte units
    assert layers[0].weight.grad.data_ptr() == buckets.flat.data_ptr()
    assert layers[0].bias.grad.data_ptr() == buckets.flat[24:].data_ptr()
    assert layers[1].weight.grad.data_ptr() == buckets.flat[30:].data_ptr()
    layers[0].weight_grad_out.fill_(3.0)
    assert torch.all(layers[0].weight.grad == 3.0)
    layers[0].weight.grad = None
    buckets.zero_grad()
    assert layers[0].weight.grad.data_ptr() == buckets.flat.data_ptr()


def test_narrow_exchange_dtype_needs_cuda():
    layer = attorch_b200.Linear(4, 6, device='cpu')
    with pytest.raises(RuntimeError, match='no CPU path'):
        GradientBuckets([layer], grad_dtype=torch.bfloat16)


def _leaving_worker(rank: int, world_size: int, port: int, result_queue) -> None:
    """Rank 1 leaves between steps; rank 0's next collective must end with an error, not hang."""
    import datetime
    os.environ['MASTER_ADDR'] = '127.0.0.1'
    os.environ['MASTER_PORT'] = str(port)
    dist.init_process_group('gloo', rank=rank, world_size=world_size, timeout=datetime.timedelta(seconds=5))
    layer = attorch_b200.Linear(8, 4, device='cpu')
    buckets = GradientBuckets([layer], overlap=False)
    layer.weight_grad_out.fill_(float(rank + 1))
    layer.bias_grad_out.fill_(1.0)
    buckets.finish()                                   # step 1: both ranks take part
    assert torch.all(layer.weight.grad == 3.0)
    if rank == 1:
        # Leaves between steps with nothing in flight (no destroy_process_group: it is gone).
        result_queue.put(('left', rank))
        result_queue.close()
        result_queue.join_thread()
        os._exit(0)
    try:
        layer.weight_grad_out.fill_(1.0)
        buckets.finish()                               # step 2: the peer is gone
        result_queue.put(('no error', rank))
    except Exception as error:                         # gloo reports the lost peer or the time-out
        result_queue.put(('error', type(error).__name__))
    result_queue.close()
    result_queue.join_thread()
    os._exit(0)


def test_rank_leaving_between_steps_ends_the_next_collective_with_an_error():
    ctx = mp.get_context('spawn')
    queue = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_leaving_worker, args=(r, 2, port, queue)) for r in range(2)]
    for p in procs:
        p.start()
    results = dict()
    for _ in range(2):
        kind, what = queue.get(timeout=120)
        results[kind] = what
    for p in procs:
        p.join(timeout=60)
    assert 'left' in results and 'error' in results, results
