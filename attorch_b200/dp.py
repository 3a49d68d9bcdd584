"""
Data-parallel training step for models made of ``attorch_b200.Linear`` layers.

The reference has no distributed code.  This harness covers the one pattern the fused linear layer
needs at scale: one process per GPU, the batch (token) dimension split evenly across ranks, weights
replicated, and a SUM all-reduce of every layer's ``dW`` / ``db`` - the only collective, issued with
``torch.distributed`` (NCCL over NVLink / NVSwitch on GPUs, gloo on CPUs for tests).

Each layer's kernels write its weight and bias gradient straight into a slice of one flat bucket
(no copy), and every parameter's ``.grad`` is a view of that bucket, so after ``finish()`` an
optimizer reads the sum over ranks in place.  As soon as the kernels that produce a slice are
enqueued the slice is all-reduced on a side stream while the layer's ``dX`` product - and the
backward of the layers before it - still run on the compute stream.  Because the upstream gradient
is given per token, SUM reproduces the single-GPU full-batch gradient.

The exchange may use a narrower type than the parameters (``grad_dtype``): under bf16 autocast with
fp32 master weights the kernels then write ``dW`` / ``db`` in bf16, the all-reduce moves half the
bytes, and the result is widened into the fp32 ``.grad`` on the side stream.  That is the
reference's own arithmetic (its backward computes ``dW`` in the autocast dtype,
attorch/linear_layer.py:152-156, and the engine casts it to the parameter's dtype).

Two transports carry the exchange.  ``'nccl'``: ``torch.distributed.all_reduce``.  ``'multimem'``:
the library's own kernel (``ab200_multimem_all_reduce``), which lets the NVSwitch do the additions
through an NVLink multicast mapping of the bucket (allocated with
``torch.distributed._symmetric_memory``); it needs only a handful of SMs, so the GEMMs that run
beside it keep almost all of them, and being an ordinary kernel it can be captured in a CUDA graph
together with the rest of the step.

A step that is replayed from CUDA graphs cannot issue NCCL calls from inside backward; for it the
harness can hold back the first layer's ``dX`` (``defer_first_input_grad``): the step becomes "graph 1:
forward and backward without that product", ``start_exchange()`` (one all-reduce of the whole bucket on
the side stream), "graph 2: ``run_deferred()``", ``finish()`` - the exchange hides behind the one GEMM
nothing else waits for.
"""

from typing import Iterable, List, Optional

import torch
import torch.distributed as dist
from torch import Tensor

from . import _lib
from . import linear_layer as _layer
from .linear_layer import Linear

_DTYPE_IDS = {torch.float32: _lib.F32, torch.float16: _lib.F16, torch.bfloat16: _lib.BF16}


def shard_rows(tensor: Tensor, rank: int, world_size: int) -> Tensor:
    """Contiguous block of rows ``rank`` owns when dim 0 is split evenly over ``world_size`` ranks."""
    rows = tensor.shape[0]
    if rows % world_size != 0:
        raise ValueError(f'{rows} rows do not split evenly over {world_size} ranks')
    per_rank = rows // world_size
    return tensor[rank * per_rank:(rank + 1) * per_rank]


class _MultimemBucket:
    """
    A gradient bucket every rank maps through one NVLink multicast object, plus the flag block the
    library's all-reduce kernel synchronises the ranks with.  PyTorch's symmetric-memory allocator
    provides the mappings (plumbing); the collective itself is ``ab200_multimem_all_reduce``.
    """
    def __init__(self, numel: int, dtype: torch.dtype, device: torch.device, group, ctas: int) -> None:
        import torch.distributed._symmetric_memory as symm_mem
        group = group if group is not None else dist.group.WORLD
        lib = _lib.load()
        self.flat = symm_mem.empty(numel, dtype=dtype, device=device)
        self.flat.zero_()
        handle = symm_mem.rendezvous(self.flat, group)
        if not handle.multicast_ptr:
            raise RuntimeError('NVLink multicast is not available for this group of devices')
        self.flags = symm_mem.empty(lib.ab200_collective_flag_bytes() // 4, dtype=torch.int32, device=device)
        self.flags.zero_()
        flag_handle = symm_mem.rendezvous(self.flags, group)
        self.multicast_ptr = int(handle.multicast_ptr)
        self.flag_blocks = int(flag_handle.buffer_ptrs_dev)      # device array of the ranks' flag blocks
        self.rank, self.world_size = int(handle.rank), int(handle.world_size)
        self.dtype, self.device, self.ctas = dtype, device, ctas
        self.element_size = self.flat.element_size()
        self._handles = (handle, flag_handle)                    # keep the mappings alive
        # Every rank's flags are zero before any rank's first kernel signals them.
        torch.cuda.synchronize(device)
        dist.barrier(group=group)

    def can_reduce(self, begin: int, end: int) -> bool:
        return (begin * self.element_size) % 16 == 0 and ((end - begin) * self.element_size) % 16 == 0

    def all_reduce(self, begin: int, end: int) -> None:
        stream = torch.cuda.current_stream(self.device).cuda_stream
        with torch.cuda.device(self.device):
            status = _layer._stream_scratch(self.device)['status']
        _lib.check(_lib.load().ab200_multimem_all_reduce(
            self.multicast_ptr + begin * self.element_size, end - begin, _DTYPE_IDS[self.dtype], self.rank,
            self.world_size, self.flag_blocks, self.ctas, status.data_ptr(), stream),
            'ab200_multimem_all_reduce')


class GradientBuckets:
    """
    One flat gradient buffer per model; every Linear gets views of it as its ``dW`` / ``db``
    destinations, its parameters' ``.grad`` alias it, and a callback all-reduces the layer's slice.

    Args:
        layers: The Linear layers, in forward order.
        process_group: Group to reduce over; None for the default group.  With a world size of 1
            (or torch.distributed not initialised) no collective is issued.
        overlap: Issue each layer's all-reduce on a side stream as soon as its gradients are
            enqueued (CUDA only); otherwise reduce everything in ``finish``.
        comm_sms: SMs left free for the collective while it overlaps the remaining GEMMs of
            backward: the persistent GEMM kernels would otherwise hold every SM and the all-reduce
            would only start once they end.
        dw_chunks: Each layer's dW is computed and exchanged in this many blocks of rows, which
            widens the window the exchange can hide in from "dX" to "the rest of dW, then dX".
        defer_first_input_grad: The first layer's dX - the last product of backward, which nothing
            inside backward consumes - is not launched by backward but by ``run_deferred()``.  A
            step can then be two replayable pieces with the exchange started in between:
            forward + backward without that dX; ``start_exchange()``; ``run_deferred()``;
            ``finish()``.  The input's ``.grad`` is complete only after ``run_deferred()``.
        grad_dtype: Element type the gradients are computed and exchanged in; None for the
            parameters' own.  If it differs, ``.grad`` (in the parameters' dtype) receives the
            widened sum after the exchange.
        exchange: False builds the same buckets without any collective, as if the world size were 1
            (to time or test a rank's local step while other ranks exist).
        transport: ``'nccl'``, ``'multimem'`` (raises where NVLink multicast is not available) or
            ``'auto'`` (multimem where available, else NCCL); see the module docstring.
        comm_ctas: CTAs of the multimem kernel (it also sets ``comm_sms`` for that transport).
    """
    def __init__(self, layers: Iterable[Linear], process_group=None, overlap: bool = True,
                 comm_sms: int = 16, dw_chunks: int = 2, defer_first_input_grad: bool = False,
                 grad_dtype: Optional[torch.dtype] = None, exchange: bool = True, transport: str = 'nccl',
                 comm_ctas: int = 8) -> None:
        self.layers: List[Linear] = list(layers)
        self.group = process_group
        self.world_size = dist.get_world_size(process_group) if (dist.is_initialized() and exchange) else 1
        first = self.layers[0].weight
        self.device = first.device
        self.dtype = first.dtype
        self.grad_dtype = grad_dtype if grad_dtype is not None else self.dtype
        total = sum(layer.weight.numel() + (layer.bias.numel() if layer.bias is not None else 0)
                    for layer in self.layers)
        # What the kernels write and the collective reduces (padded to whole 16-byte units).
        elt = torch.empty(0, dtype=self.grad_dtype).element_size()
        total = -(-total * elt // 16) * 16 // elt
        self.transport = 'nccl'
        self._multimem = None
        if transport not in ('nccl', 'multimem', 'auto'):
            raise ValueError(f"transport must be 'nccl', 'multimem' or 'auto', not {transport!r}")
        if transport != 'nccl' and self.world_size > 1 and self.device.type == 'cuda':
            failure = None
            try:
                self._multimem = _MultimemBucket(total, self.grad_dtype, self.device, process_group, comm_ctas)
            except Exception as error:
                failure = error
            # All ranks use the same transport: one that could not set the mapping up sends everybody to NCCL.
            agreed = torch.tensor([0 if failure is None else 1], dtype=torch.int32, device=self.device)
            dist.all_reduce(agreed, op=dist.ReduceOp.MAX, group=process_group)
            if int(agreed.item()) == 0:
                self.transport = 'multimem'
                comm_sms = comm_ctas
            else:
                self._multimem = None
                if transport == 'multimem':
                    raise RuntimeError('NVLink multicast transport unavailable on at least one rank') from failure
        self.flat = (self._multimem.flat if self._multimem is not None else
                     torch.zeros(total, dtype=self.grad_dtype, device=self.device))
        # What .grad aliases: the same buffer, or a second one in the parameters' dtype.
        self.widen = self.grad_dtype is not self.dtype
        self.flat_grad = torch.zeros(total, dtype=self.dtype, device=self.device) if self.widen else self.flat
        if self.widen and self.device.type != 'cuda':
            raise RuntimeError('a narrower exchange dtype needs the CUDA cast kernel: no CPU path')
        self.slices: List[Tensor] = []
        self._offsets: List[int] = []
        self.overlap = overlap and self.device.type == 'cuda' and self.world_size > 1
        self.comm_sms = comm_sms
        self.comm_stream = torch.cuda.Stream(self.device) if self.overlap else None
        self._pending: List[torch.cuda.Event] = []
        self._deferred: List = []
        self._grad_views: List = []
        if defer_first_input_grad:
            self.layers[0].defer_input_grad = self._deferred.append
        offset = 0
        for index, layer in enumerate(self.layers):
            if layer.weight.dtype is not self.dtype:
                raise TypeError('all layers of one bucket must share a parameter dtype')
            begin = offset
            n = layer.weight.numel()
            layer.weight_grad_out = self.flat[offset:offset + n].view_as(layer.weight)
            weight_grad = self.flat_grad[offset:offset + n].view_as(layer.weight)
            offset += n
            bias_grad = None
            if layer.bias is not None:
                n = layer.bias.numel()
                layer.bias_grad_out = self.flat[offset:offset + n]
                bias_grad = self.flat_grad[offset:offset + n]
                offset += n
            self.slices.append(self.flat[begin:offset])
            self._offsets.append(begin)
            self._grad_views.append((weight_grad, bias_grad))
            layer.grad_ready = self._make_callback(index)
            layer.dw_chunks = dw_chunks if self.overlap else 1
        self.bind_grads()

    def bind_grads(self) -> None:
        """
        Points every parameter's ``.grad`` at its view of the bucket.  Backward writes the bucket
        through the layer's destination buffers and returns no gradient of its own for them, so
        these aliases are what an optimizer reads (after ``finish()``).
        """
        for layer, (weight_grad, bias_grad) in zip(self.layers, self._grad_views):
            layer.weight.grad = weight_grad
            if layer.bias is not None:
                layer.bias.grad = bias_grad

    def _make_callback(self, index: int):
        def grad_ready(block: int = 0, blocks: int = 1) -> None:
            if not self.overlap:
                return
            # Block i of n covers rows [i K / n, (i + 1) K / n) of dW, contiguous in the bucket; the
            # bias gradient, which follows dW in the bucket, travels with the last block.
            layer = self.layers[index]
            whole = self.slices[index]
            per_block = layer.weight.numel() // blocks
            begin = block * per_block
            end = (block + 1) * per_block if block + 1 < blocks else whole.numel()
            self._reduce_async(self._offsets[index] + begin, self._offsets[index] + end)
        return grad_ready

    def _widen(self, begin: int, end: int) -> None:
        """flat_grad[begin:end] <- flat[begin:end] in the parameters' dtype, on the current stream."""
        src, dst = self.flat[begin:end], self.flat_grad[begin:end]
        _lib.check(_lib.load().ab200_cast_2d(
            src.data_ptr(), dst.data_ptr(), 1, end - begin, end - begin, 1,
            _DTYPE_IDS[self.grad_dtype], _DTYPE_IDS[self.dtype],
            torch.cuda.current_stream(self.device).cuda_stream), 'ab200_cast_2d')

    def _all_reduce(self, begin: int, end: int) -> None:
        """SUM over ranks of flat[begin:end], in place, on the current stream."""
        if self._multimem is not None and self._multimem.can_reduce(begin, end):
            self._multimem.all_reduce(begin, end)
        else:
            dist.all_reduce(self.flat[begin:end], op=dist.ReduceOp.SUM, group=self.group)

    def _reduce_async(self, begin: int, end: int) -> None:
        ready = torch.cuda.Event()
        ready.record(torch.cuda.current_stream(self.device))
        with torch.cuda.stream(self.comm_stream):
            self.comm_stream.wait_event(ready)
            self._all_reduce(begin, end)
            if self.widen:
                self._widen(begin, end)
            done = torch.cuda.Event()
            done.record(self.comm_stream)
        self._pending.append(done)
        # The GEMMs enqueued from here to finish() run beside the collective.
        _layer.set_reserved_sms(self.device.index, self.comm_sms)

    def start_exchange(self) -> None:
        """
        Starts the all-reduce of the whole bucket on the side stream, ordered after everything enqueued
        so far on the current stream (for steps that run backward with ``overlap=False`` and
        ``defer_first_input_grad=True``); ``finish()`` waits for it.
        """
        if self.world_size == 1 or self.device.type != 'cuda':
            return
        if self.comm_stream is None:
            self.comm_stream = torch.cuda.Stream(self.device)
        ready = torch.cuda.Event()
        ready.record(torch.cuda.current_stream(self.device))
        with torch.cuda.stream(self.comm_stream):
            self.comm_stream.wait_event(ready)
            self._all_reduce(0, self.flat.numel())
            if self.widen:
                self._widen(0, self.flat.numel())
            done = torch.cuda.Event()
            done.record(self.comm_stream)
        self._pending.append(done)

    def exchange_sms(self) -> int:
        """SMs a GEMM should leave free while it runs beside the exchange (0: none)."""
        return self.comm_sms if (self.device.type == 'cuda' and self.world_size > 1) else 0

    def run_deferred(self, rows=None, keep: bool = False, reserve_sms: int = 0) -> None:
        """
        Launches the products ``defer_first_input_grad`` held back, on the current stream: all of
        their rows, or rows ``[rows[0], rows[1])`` only (``keep=True`` leaves them registered for a
        further call with the remaining rows).  ``reserve_sms`` SMs are left free for the exchange
        that runs beside these launches.
        """
        previous = _layer.set_reserved_sms(self.device.index, reserve_sms) if self.device.type == 'cuda' else 0
        try:
            for launch in self._deferred:
                if rows is None:
                    launch()
                else:
                    launch(rows[0], rows[1])
        finally:
            if self.device.type == 'cuda':
                _layer.set_reserved_sms(self.device.index, previous)
        if not keep:
            self._deferred.clear()

    def finish(self) -> None:
        """
        Completes the gradient exchange of one step: after it returns (in stream order on the
        current stream) every parameter's ``.grad`` holds the sum over ranks.
        """
        if self._pending:
            current = torch.cuda.current_stream(self.device)
            for done in self._pending:
                current.wait_event(done)
            self._pending.clear()
            if self.overlap:
                _layer.set_reserved_sms(self.device.index, 0)
            return
        if self.world_size > 1:
            self._all_reduce(0, self.flat.numel())
        if self.widen:
            self._widen(0, self.flat.numel())

    def zero_grad(self) -> None:
        """
        Prepares the next step.  The kernels overwrite the bucket (they do not accumulate), so
        nothing needs clearing; the ``.grad`` aliases are kept, or restored if something dropped them.
        """
        for layer, (weight_grad, bias_grad) in zip(self.layers, self._grad_views):
            grad = layer.weight.grad
            if grad is None or grad.data_ptr() != weight_grad.data_ptr():
                layer.weight.grad = weight_grad
            if layer.bias is not None:
                grad = layer.bias.grad
                if grad is None or grad.data_ptr() != bias_grad.data_ptr():
                    layer.bias.grad = bias_grad
