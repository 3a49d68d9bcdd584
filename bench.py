"""
Benchmark of the fused linear layer (forward + backward) on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload c2|c3|c4|c5|act|ce] [--impl reference]

For N > 1 launch one rank per GPU with torchrun (RANK / LOCAL_RANK / WORLD_SIZE / MASTER_* from the
environment).  Rank 0 prints one JSON line, last.

Workloads (synthetic, seeded; shapes of the reference configurations this path is quoted on):
  c2  attorch.Linear 4096 -> 4096, bias, gelu, under bf16 autocast with fp32 parameters and fp32
      input; 8192 tokens per GPU (weak scaling: the global batch is 8192 * N); forward + backward
      (dX, dW, db); with N > 1 dW / db are SUM-all-reduced every step, overlapped with dX.
  c5  two layers 8192 -> 8192 (gelu + bias, then bias), bf16 parameters, global batch 65536 tokens
      split over the N GPUs (strong scaling), same all-reduce.
  c3  transformer MLP pair 4096 -> 14336 (silu) -> 4096, no biases, bf16, 16384 tokens per GPU.
  c4  skinny forward only, fp16, 8192 -> 28672, M in {1, 8, 32, 128}: prints weight-read GB/s.
  act standalone activation layer (GELU, drop_p = 0.1, bf16, 32768 x 4096 elements) and gated linear
      unit (silu, bf16, 16384 x 2*14336): GB/s.
  ce  cross-entropy loss of bf16 logits [8192, 50304], forward and backward: GB/s.

One "step" is one forward + backward of the workload on one batch.  ``value`` is the whole-job
TFLOP/s at 6 * M * K * N floating-point operations per layer and step with the inputs resident in
HBM; ``e2e`` is the same through the same module with the step's input copied from pinned host
memory and the output and the bias gradient read back every step (copies on side streams).
The default run (workload c2) adds sub-records to the same line: ``c5`` (its step at this N, and at
N > 1 the same 65536 tokens on one GPU for the strong-scaling efficiency), ``dp_parity`` (all-reduced
gradients against the full-batch gradients of the gathered shards), ``collectives`` (all-reduce times),
and at N = 1 ``torch_gpu_baseline`` (torch.nn.Linear + gelu and bare matmuls on the same GPU), ``c3``
and ``c4``.  ``--impl reference`` times the CPU computation the reference's tests compare against
(torch.nn.Linear + activation, all host cores) on the same batch.
"""

import argparse
import json
import os
import re
import socket
import statistics
import sys
import tempfile
import threading
import time
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

PEAK_FALLBACK = {'hbm_gbs': 6650.0, 'bf16_tflops': 1590.0, 'bf16_tflops_sustained': 1400.0}

WORKLOADS = {
    'c2': dict(layers=[(4096, 4096, 'gelu', True)], tokens_per_gpu=8192, global_tokens=None,
               param_dtype=torch.float32, input_dtype=torch.float32, autocast=torch.bfloat16,
               scaling='weak'),
    'c5': dict(layers=[(8192, 8192, 'gelu', True), (8192, 8192, None, True)], tokens_per_gpu=None,
               global_tokens=65536, param_dtype=torch.bfloat16, input_dtype=torch.bfloat16,
               autocast=None, scaling='strong'),
    'c3': dict(layers=[(4096, 14336, 'silu', False), (14336, 4096, None, False)], tokens_per_gpu=16384,
               global_tokens=None, param_dtype=torch.bfloat16, input_dtype=torch.bfloat16,
               autocast=None, scaling='weak'),
}
# The skinny forward-only workload c4 is HBM-bound: see skinny_forward().

DTYPE_NAMES = {torch.float32: 'fp32', torch.bfloat16: 'bf16', torch.float16: 'fp16'}


def measured_peaks():
    path = ROOT / 'MEASURED_PEAKS.json'
    if path.exists():
        data = json.loads(path.read_text())
        return {k: float(data[k]) for k in PEAK_FALLBACK}, 'measured'
    return dict(PEAK_FALLBACK), 'fallback'


def profiled_dram_bytes(summary: str = 'c2_kernel_fwd.md'):
    """
    DRAM bytes per launch (read + written, mean over the captured launches) of the forward GEMM of
    workload c2, read from the committed summary of its ncu capture; None if the file or the lines
    are missing.
    """
    path = ROOT / 'profiles' / summary
    if not path.exists():
        return None
    total = 0.0
    for key in ('dram__bytes_read.sum', 'dram__bytes_write.sum'):
        match = re.search(re.escape(key) + r' \[(\w+)\]: ([^\n]+)', path.read_text())
        if match is None:
            return None
        scale = {'Mbyte': 1e6, 'Gbyte': 1e9, 'Kbyte': 1e3, 'byte': 1.0}.get(match.group(1))
        try:
            values = [float(v) for v in match.group(2).split('|')]
        except ValueError:
            return None
        if scale is None or not values:
            return None
        total += scale * sum(values) / len(values)
    return total


class ClockSampler:
    """Samples SM clock and throttle reasons through NVML while the timed region runs."""
    def __init__(self, index: int) -> None:
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop = threading.Event()
        self._thread = None
        try:
            if index < 0:
                raise RuntimeError('only rank 0 samples')
            import pynvml
            pynvml.nvmlInit()
            self._nvml = pynvml
            self._handle = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self._handle, pynvml.NVML_CLOCK_SM)
        except Exception:
            self._nvml = None

    def _run(self) -> None:
        nv = self._nvml
        names = {'hw_slowdown': 'nvmlClocksEventReasonHwSlowdown',
                 'hw_thermal_slowdown': 'nvmlClocksEventReasonHwThermalSlowdown',
                 'sw_thermal_slowdown': 'nvmlClocksEventReasonSwThermalSlowdown',
                 'sw_power_cap': 'nvmlClocksEventReasonSwPowerCap'}
        fallback = {'hw_slowdown': 0x8, 'hw_thermal_slowdown': 0x40, 'sw_thermal_slowdown': 0x20,
                    'sw_power_cap': 0x4}
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self._handle, nv.NVML_CLOCK_SM))
                try:
                    mask = nv.nvmlDeviceGetCurrentClocksEventReasons(self._handle)
                except Exception:
                    mask = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self._handle)
                for name, attr in names.items():
                    bit = getattr(nv, attr, fallback[name])
                    if mask & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            time.sleep(0.005)

    def __enter__(self):
        if self._nvml is not None:
            self._thread = threading.Thread(target=self._run, daemon=True)
            self._thread.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        if self._thread is not None:
            self._thread.join()

    def summary(self):
        if not self.samples:
            return {'sm_mhz': None, 'sm_max_mhz': self.max_mhz, 'reasons': ['unavailable']}
        return {'sm_mhz': statistics.median(self.samples), 'sm_max_mhz': self.max_mhz,
                'reasons': sorted(self.reasons), 'samples': len(self.samples)}


class CollectiveLog:
    """
    NCCL writes its INFO log to standard output, where rank 0's JSON line has to be the last line.
    For the life of this object file descriptor 1 points to a temporary file instead; ``close()``
    puts standard output back, copies the NCCL lines that say which algorithm ran to standard error
    and returns them.
    """
    PATTERN = re.compile(r'AllReduce: (\d+) Bytes -> Algo (\w+) proto (\w+) channel\{Lo\.\.Hi\}=\{(\d+)\.\.(\d+)\}')

    def __init__(self) -> None:
        # INFO level with the INIT and TUNING subsystems: the latter logs the algorithm, protocol and
        # channel count of every collective.  Whatever the launcher asked for on top of that is kept.
        if os.environ.get('NCCL_DEBUG', '').upper() not in ('INFO', 'TRACE'):
            os.environ['NCCL_DEBUG'] = 'INFO'
        subsys = [s for s in os.environ.get('NCCL_DEBUG_SUBSYS', '').split(',') if s]
        if not any(s.upper() == 'ALL' for s in subsys):
            for wanted in ('INIT', 'TUNING'):
                if not any(s.upper() == wanted for s in subsys):
                    subsys.append(wanted)
        os.environ['NCCL_DEBUG_SUBSYS'] = ','.join(subsys)
        sys.stdout.flush()
        self._saved = os.dup(1)
        self._file = tempfile.TemporaryFile(mode='w+b')
        os.dup2(self._file.fileno(), 1)

    def _text(self) -> str:
        sys.stdout.flush()
        self._file.seek(0)
        chunks = [self._file.read().decode(errors='replace')]
        self._file.seek(0, os.SEEK_END)
        # A launcher may have sent the log to a file of its own.
        pattern = os.environ.get('NCCL_DEBUG_FILE')
        if pattern:
            path = pattern.replace('%h', socket.gethostname()).replace('%p', str(os.getpid()))
            try:
                chunks.append(Path(path).read_text(errors='replace'))
            except OSError:
                pass
        return '\n'.join(chunks)

    def all_reduce_choice(self, nbytes: int):
        """(algorithm, protocol, channels) NCCL logged for the all-reduce closest in size to nbytes."""
        best = None
        for match in self.PATTERN.finditer(self._text()):
            size = int(match.group(1))
            if best is None or abs(size - nbytes) < abs(best[0] - nbytes):
                best = (size, match.group(2), match.group(3), int(match.group(5)) - int(match.group(4)) + 1)
        return None if best is None or best[0] < nbytes // 4 else best[1:]

    def close(self, echo: bool) -> str:
        text = self._text()
        sys.stdout.flush()
        os.dup2(self._saved, 1)
        os.close(self._saved)
        self._file.close()
        keep = [line for line in text.splitlines()
                if re.search(r'NVLS|nvls|-> Algo|coll channels|nranks|Connected all', line)]
        seen, tail = set(), []
        for line in keep:
            key = re.sub(r'^\S+ ', '', line)
            if key not in seen:
                seen.add(key)
                tail.append(line)
        tail = tail[-24:]
        if echo:
            for line in tail:
                print(line, file=sys.stderr)
        return '\n'.join(tail)


def flops_per_step(spec, tokens):
    return sum(6.0 * tokens * k * n for (k, n, _, _) in spec['layers'])


def cpu_arm(spec, tokens, steps, warmup):
    """torch.nn.Linear + activation forward + backward in fp32 on all host cores, on `tokens` rows."""
    from oracle.cpu_baseline import time_torch_cpu_linear
    seconds, threads = 0.0, 1
    for (k, n, act, bias) in spec['layers']:
        r = time_torch_cpu_linear(tokens, k, n, act, bias, None, steps, warmup)
        seconds += r['seconds_per_step']
        threads = r['threads']
    return seconds, threads


def run_reference(args, spec, world_size, rank):
    """CPU arm: the whole batch of one GPU's step per CPU step (same configuration as the GPU arm)."""
    if rank != 0:
        return
    tokens = args.tokens or spec['tokens_per_gpu'] or spec['global_tokens']
    seconds, threads = cpu_arm(spec, tokens, args.steps, min(args.warmup, 3))
    tflops = flops_per_step(spec, tokens) / seconds / 1e12
    sample = (f'all {tokens} rows of one GPU\'s batch per step, torch.nn.Linear + activation fwd+bwd in fp32 '
              f'on {threads} host threads')
    line = {
        'impl': 'reference', 'metric': 'linear_fwd_bwd_tflops', 'value': tflops, 'unit': 'TFLOP/s',
        'n_gpus': world_size, 'steps': args.steps, 'warmup': args.warmup,
        'ms_per_step': seconds * 1e3, 'higher_is_better': True, 'scaling': spec['scaling'],
        'vs_baseline': None, 'dtype': 'f32', 'data': 'synthetic',
        'config': {'workload': args.workload,
                   'layers': [f'{k}->{n} act={act} bias={bias}' for (k, n, act, bias) in spec['layers']],
                   'tokens_per_gpu': tokens, 'sample': sample},
        'cpu_baseline': {'value': tflops, 'unit': 'TFLOP/s', 'cores': threads, 'kind': 'port',
                         'sample': sample},
        'e2e': {'value': tflops, 'unit': 'TFLOP/s', 'h2d_bytes_per_step': 0, 'd2h_bytes_per_step': 0},
        'gpu_launches': 0,
    }
    print(json.dumps(line), flush=True)


def kernel_launcher(spec, tokens, device, lib, which='fwd'):
    """
    Returns (launch, work, unit): `launch()` enqueues one kernel of the workload's first layer through
    the C ABI exactly as the layer launches it, on the current stream.  `which`:
      fwd      forward tcgen05 GEMM, X[M, K] * W[K, N] with bias, activation, saved act'(Z)
      dx       backward tcgen05 GEMM dX = dZ * W^T
      dw       backward tcgen05 GEMM dW = X^T * dZ
      act_bwd  dZ = dY * saved act'(Z) with the bias-gradient column sums
    `work` is the algorithmic work of one launch: floating-point operations for the GEMMs, bytes
    (dY and Z read, dZ written) for act_bwd.
    """
    from attorch_b200 import _lib
    from attorch_b200.acts import act_id, parse_act_func
    k0, n0, act0, _ = spec['layers'][0]
    op_dtype = spec['autocast'] or spec['param_dtype']
    grad_dtype = spec['param_dtype']
    ids = {torch.float32: 0, torch.float16: 1, torch.bfloat16: 2}
    xo = torch.randn(tokens, k0, device=device).to(op_dtype)
    wo = (torch.randn(k0, n0, device=device) / k0 ** 0.5).to(op_dtype)
    bo = torch.randn(n0, device=device).to(grad_dtype)
    yo = torch.empty(tokens, n0, device=device, dtype=op_dtype)
    zo = torch.randn(tokens, n0, device=device).to(op_dtype)
    dyo = (torch.randn(tokens, n0, device=device) * 0.01).to(op_dtype)
    dzo = torch.randn(tokens, n0, device=device).to(op_dtype)
    dxo = torch.empty(tokens, k0, device=device, dtype=spec['input_dtype'])
    dwo = torch.empty(k0, n0, device=device, dtype=grad_dtype)
    dbo = torch.empty(n0, device=device, dtype=grad_dtype)
    ws = torch.empty(max(lib.ab200_act_backward_workspace_bytes(tokens, n0), 16), dtype=torch.uint8, device=device)
    gws_bytes = max(lib.ab200_gemm_workspace_bytes(tokens, n0, k0), lib.ab200_gemm_workspace_bytes(k0, n0, tokens),
                    lib.ab200_gemm_workspace_bytes(tokens, k0, n0), 16)
    gws = torch.empty(gws_bytes, dtype=torch.uint8, device=device)
    status = torch.zeros(1, dtype=torch.int32, device=device)
    dt_id = ids[op_dtype]
    name, param = parse_act_func(act0)
    stream = torch.cuda.current_stream().cuda_stream
    keep = (xo, wo, bo, yo, zo, dyo, dzo, dxo, dwo, dbo, ws, gws, status)
    flags = _lib.FLAG_FORCE_TCGEN05 | _lib.FLAG_NO_STREAMK
    # As the layer does by default: forward saves act'(Z), backward multiplies by it.
    fwd_flags = flags | (_lib.FLAG_SAVE_DERIVATIVE if name is not None else 0)
    bwd_act = _lib.ACT_SAVED_DERIVATIVE if name is not None else 0
    gemm_flops = 2.0 * tokens * k0 * n0

    def fwd():
        _lib.check(lib.ab200_linear_forward(
            xo.data_ptr(), wo.data_ptr(), bo.data_ptr(), zo.data_ptr(), yo.data_ptr(), tokens, k0, n0,
            k0, 1, n0, 1, n0, n0, dt_id, dt_id, ids[bo.dtype], act_id(name), param or 0.0, gws.data_ptr(), gws_bytes,
            status.data_ptr(), stream, fwd_flags), 'ab200_linear_forward')
        return keep

    def dx():
        _lib.check(lib.ab200_linear_backward_input(
            dzo.data_ptr(), wo.data_ptr(), dxo.data_ptr(), tokens, k0, n0, n0, 1, n0, 1, k0, dt_id,
            ids[dxo.dtype], gws.data_ptr(), gws_bytes, status.data_ptr(), stream, flags),
            'ab200_linear_backward_input')
        return keep

    def dw():
        _lib.check(lib.ab200_linear_backward_weight(
            xo.data_ptr(), dzo.data_ptr(), dwo.data_ptr(), tokens, k0, n0, k0, 1, n0, 1, n0, dt_id,
            ids[dwo.dtype], gws.data_ptr(), gws_bytes, status.data_ptr(), stream, flags),
            'ab200_linear_backward_weight')
        return keep

    def act_bwd():
        _lib.check(lib.ab200_act_backward(
            dyo.data_ptr(), zo.data_ptr(), dzo.data_ptr(), dbo.data_ptr(), tokens, n0, n0, n0, n0, dt_id,
            ids[dbo.dtype], bwd_act, param or 0.0, ws.data_ptr(), ws.numel(), stream),
            'ab200_act_backward')
        return keep

    if which == 'act_bwd':
        return act_bwd, 3.0 * tokens * n0 * dyo.element_size(), 'bytes'
    return {'fwd': fwd, 'dx': dx, 'dw': dw}[which], gemm_flops, 'flops'


def event_time(fn, reps, warmup=3):
    """Mean milliseconds of `fn()` over `reps` back-to-back calls, CUDA events on the current stream."""
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0.record()
    for _ in range(reps):
        fn()
    t1.record()
    torch.cuda.synchronize()
    return t0.elapsed_time(t1) / reps


def kernel_only(args, spec, tokens, device, lib):
    """A few launches of one kernel and nothing else: the target of ncu captures."""
    launch, work, unit = kernel_launcher(spec, tokens, device, lib, args.kernel_only)
    ms = event_time(launch, args.steps, max(args.warmup, 1))
    rate = {'tflops': work / (ms * 1e-3) / 1e12} if unit == 'flops' else {'gbs': work / (ms * 1e-3) / 1e9}
    print(json.dumps({'kernel_only': args.kernel_only, 'tokens': tokens, 'kernel_ms': ms, **rate}), flush=True)


def skinny_forward(steps, warmup, device, lib):
    """
    Skinny forward-only workload c4: y = x @ W for fp16 x [M, 8192], W [8192, 28672], no bias, no
    activation, under torch.no_grad(), through the module.  HBM-bound: the score is algorithmic bytes
    2 * (K * N + M * K + M * N) over the CUDA-event time, in GB/s.  W (448 MiB) exceeds the L2, so
    back-to-back launches are cold.
    """
    import attorch_b200
    from attorch_b200 import _lib
    K, N = 8192, 28672
    peaks, peak_source = measured_peaks()
    layer = attorch_b200.Linear(K, N, bias=False, device=device, dtype=torch.float16)
    with torch.no_grad():
        layer.weight.normal_(0, 0.02)
    rows = []
    for m in (1, 8, 32, 128):
        x = torch.randn(m, K, device=device, dtype=torch.float16)
        with torch.no_grad():
            call = lambda: layer(x)
            replayed = False
            try:
                # Replayed from a CUDA graph: at 80 us per call the host side of an eager call
                # (Python, three launches for the stream-K route) would otherwise set the pace.
                side = torch.cuda.Stream(device)
                side.wait_stream(torch.cuda.current_stream())
                with torch.cuda.stream(side):
                    for _ in range(3):
                        layer(x)
                torch.cuda.current_stream().wait_stream(side)
                torch.cuda.synchronize()
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph):
                    out = layer(x)
                call, replayed = graph.replay, True
            except Exception as error:
                print(f'c4: CUDA graph capture failed, timing eager calls ({error})', file=sys.stderr)
                torch.cuda.synchronize()
            ms = event_time(call, steps, max(warmup, 3))
        nbytes = 2.0 * (K * N + m * K + m * N)
        path = {_lib.PATH_STREAMK: 'memset + swap-AB stream-K tcgen05 + finish',
                _lib.PATH_TCGEN05: 'one wave of whole 128 x 256 tcgen05 tiles'}.get(lib.ab200_last_path(), 'other')
        rows.append({'M': m, 'us': ms * 1e3, 'gbs': nbytes / (ms * 1e-3) / 1e9, 'path': path, 'cuda_graph': replayed,
                     'frac_of_measured_hbm': nbytes / (ms * 1e-3) / 1e9 / peaks['hbm_gbs'],
                     'frac_of_nominal_8000': nbytes / (ms * 1e-3) / 1e9 / 8000.0})
    attorch_b200.check_status()
    best = max(r['gbs'] for r in rows)
    return {'metric': 'skinny_forward_weight_read_gbs', 'value': best, 'unit': 'GB/s', 'n_gpus': 1,
            'steps': steps, 'warmup': warmup, 'higher_is_better': True, 'dtype': 'f16',
            'data': 'synthetic', 'config': {'workload': 'c4', 'K': K, 'N': N, 'rows': rows,
                                            'call': 'attorch_b200.Linear under torch.no_grad()'},
            'roofline': {'bound': 'hbm', 'achieved': best, 'peak': peaks['hbm_gbs'], 'unit': 'GB/s',
                         'frac': best / peaks['hbm_gbs'], 'traffic': None, 'peak_source': peak_source}}


def activation_layer(args, device):
    """
    The standalone activation layer with fused dropout: GELU with drop_p = 0.1 on a bf16 [32768, 4096]
    tensor (268 MB, larger than L2), forward and input gradient, timed through the C ABI (the kernels
    alone) and through attorch_b200.GELU (with the host work of the module around them).  HBM-bound:
    algorithmic bytes are 2 n e forward (read x, write y) and 3 n e backward (read dy and x, write dx).
    """
    import attorch_b200
    from attorch_b200 import _lib
    from attorch_b200.acts import act_id, parse_act_func
    lib = _lib.load()
    peaks, peak_source = measured_peaks()
    n_rows, n_cols = 32768, 4096
    n = n_rows * n_cols
    x = torch.randn(n_rows, n_cols, device=device).bfloat16()
    dy = torch.randn(n_rows, n_cols, device=device).bfloat16()
    out = torch.empty_like(x)
    act, param = act_id(parse_act_func('gelu')[0]), 0.0
    stream = torch.cuda.current_stream().cuda_stream

    def kernel_forward(flags=0):
        rc = lib.ab200_act_forward(x.data_ptr(), out.data_ptr(), n, _lib.BF16, act, param, 0.1, 7, stream, flags)
        assert rc == 0, rc

    def kernel_backward(flags=0):
        rc = lib.ab200_act_input_grad(dy.data_ptr(), x.data_ptr(), out.data_ptr(), n, _lib.BF16, act, param,
                                      0.1, 7, stream, flags)
        assert rc == 0, rc

    def kernel_forward_no_dropout():
        rc = lib.ab200_act_forward(x.data_ptr(), out.data_ptr(), n, _lib.BF16, act, param, 0.0, 0, stream, 0)
        assert rc == 0, rc

    layer = attorch_b200.GELU(drop_p=0.1)
    layer.train()
    xg = x.clone().requires_grad_(True)

    def module_step():
        layer(xg).backward(dy)
        xg.grad = None

    packed = _lib.FLAG_DROPOUT_PACKED
    results = {}
    for name, fn, nbytes in (('kernel_forward', kernel_forward, 2 * n * 2.0),
                             ('kernel_backward', kernel_backward, 3 * n * 2.0),
                             ('kernel_forward_packed_stream', lambda: kernel_forward(packed), 2 * n * 2.0),
                             ('kernel_backward_packed_stream', lambda: kernel_backward(packed), 3 * n * 2.0),
                             ('kernel_forward_no_dropout', kernel_forward_no_dropout, 2 * n * 2.0),
                             ('module_forward_backward', module_step, 5 * n * 2.0)):
        if args.only and name != args.only:
            continue
        ms = event_time(fn, args.steps, max(args.warmup, 3))
        results[name] = {'us': round(ms * 1e3, 2), 'gbs': round(nbytes / (ms * 1e-3) / 1e9, 1)}
    # Gated linear unit of the MLP pair of workload c3: silu gate over the last dimension of
    # [16384, 2 * 14336] bf16 (3 n e bytes forward, 5 n e backward for n output elements).
    del x, dy, out, xg
    rows, half = 16384, 14336
    gx = torch.randn(rows, 2 * half, device=device).bfloat16()
    gdy = torch.randn(rows, half, device=device).bfloat16()
    gy = torch.empty(rows, half, device=device, dtype=torch.bfloat16)
    gdx = torch.empty_like(gx)
    silu = act_id('silu')

    def glu_forward():
        rc = lib.ab200_glu_forward(gx.data_ptr(), gy.data_ptr(), rows, half, _lib.BF16, silu, 0.0, stream)
        assert rc == 0, rc

    def glu_backward():
        rc = lib.ab200_glu_backward(gdy.data_ptr(), gx.data_ptr(), gdx.data_ptr(), rows, half, _lib.BF16, silu, 0.0,
                                    stream)
        assert rc == 0, rc

    for name, fn, nbytes in (('glu_forward', glu_forward, 3 * rows * half * 2.0),
                             ('glu_backward', glu_backward, 5 * rows * half * 2.0)):
        if args.only and name != args.only:
            continue
        ms = event_time(fn, args.steps, max(args.warmup, 3))
        results[name] = {'us': round(ms * 1e3, 2), 'gbs': round(nbytes / (ms * 1e-3) / 1e9, 1)}
    # The same gate fused into the projection that feeds it (4096 -> 2 * 14336 on 16384 tokens, the gated
    # up-projection of the MLP pair): one kernel against projection + gated-unit kernel; TFLOP/s of the product.
    del gx, gdy, gy, gdx
    torch.cuda.empty_cache()
    if not args.only or args.only.startswith('gated'):
        tokens, k_in = 16384, 4096
        xg = torch.randn(tokens, k_in, device=device).bfloat16()
        fused = attorch_b200.GatedLinear(k_in, half, bias=False, act_func='silu', device=device, dtype=torch.bfloat16)
        plain = attorch_b200.Linear(k_in, 2 * half, bias=False, device=device, dtype=torch.bfloat16)
        gate = attorch_b200.GLU(dim=-1, act_func='silu')
        flops = 2.0 * tokens * k_in * 2 * half
        with torch.no_grad():
            for name, fn in (('gated_linear_forward_fused', lambda: fused(xg)),
                             ('gated_linear_forward_two_kernels', lambda: gate(plain(xg)))):
                if args.only and name != args.only:
                    continue
                ms = event_time(fn, args.steps, max(args.warmup, 3))
                results[name] = {'us': round(ms * 1e3, 2), 'tflops': round(flops / (ms * 1e-3) / 1e12, 1)}
    best = results.get(args.only or 'kernel_forward', {}).get('gbs', 0.0)
    print(json.dumps({'metric': 'activation_layer_gbs', 'value': best, 'unit': 'GB/s', 'n_gpus': 1,
                      'steps': args.steps, 'warmup': args.warmup, 'higher_is_better': True, 'dtype': 'bf16',
                      'data': 'synthetic',
                      'config': {'workload': 'act', 'layer': 'GELU(drop_p=0.1)', 'shape': [n_rows, n_cols],
                                 'l2': 'inputs larger than L2', **results},
                      'roofline': {'bound': 'hbm', 'achieved': best, 'peak': peaks['hbm_gbs'], 'unit': 'GB/s',
                                   'frac': best / peaks['hbm_gbs'], 'traffic': None, 'peak_source': peak_source}}),
          flush=True)


def cross_entropy_loss(args, device):
    """
    The loss after the final projection: mean cross-entropy of bf16 logits [8192 tokens, 50304 classes]
    (824 MB, larger than L2) against int64 targets, forward and backward, through the C ABI and through
    attorch_b200.CrossEntropyLoss.  HBM-bound: forward reads the logits once (n e bytes), backward reads
    them and writes the gradient (2 n e).
    """
    import attorch_b200
    from attorch_b200 import _lib
    lib = _lib.load()
    peaks, peak_source = measured_peaks()
    rows, classes = 8192, 50304
    n = rows * classes
    x = (torch.randn(rows, classes, device=device) * 2).bfloat16()
    target = torch.randint(0, classes, (rows,), device=device)
    dx = torch.empty_like(x)
    loss = torch.empty((), dtype=torch.bfloat16, device=device)
    dloss = torch.ones((), dtype=torch.bfloat16, device=device)
    lse = torch.empty(rows, dtype=torch.float32, device=device)
    ws = torch.empty(lib.ab200_cross_entropy_workspace_bytes(rows), dtype=torch.uint8, device=device)
    stream = torch.cuda.current_stream().cuda_stream

    def forward():
        _lib.check(lib.ab200_cross_entropy_forward(x.data_ptr(), target.data_ptr(), None, loss.data_ptr(), lse.data_ptr(),
                                                   rows, classes, classes, 1, _lib.BF16, 0, _lib.BF16, ws.data_ptr(),
                                                   ws.numel(), stream), 'ab200_cross_entropy_forward')

    def backward():
        _lib.check(lib.ab200_cross_entropy_backward(dloss.data_ptr(), _lib.BF16, x.data_ptr(), target.data_ptr(), None,
                                                    lse.data_ptr(), ws.data_ptr(), dx.data_ptr(), rows, classes, classes,
                                                    1, classes, _lib.BF16, 0, _lib.BF16, stream),
                   'ab200_cross_entropy_backward')

    layer = attorch_b200.CrossEntropyLoss()
    xg = x.clone().requires_grad_(True)

    def module_step():
        layer(xg, target).backward()
        xg.grad = None

    results = {}
    for name, fn, nbytes in (('kernel_forward', forward, n * 2.0), ('kernel_backward', backward, 2 * n * 2.0),
                             ('module_forward_backward', module_step, 3 * n * 2.0)):
        ms = event_time(fn, args.steps, max(args.warmup, 3))
        results[name] = {'us': round(ms * 1e3, 2), 'gbs': round(nbytes / (ms * 1e-3) / 1e9, 1)}
    best = results['kernel_forward']['gbs']
    print(json.dumps({'metric': 'cross_entropy_gbs', 'value': best, 'unit': 'GB/s', 'n_gpus': 1, 'steps': args.steps,
                      'warmup': args.warmup, 'higher_is_better': True, 'dtype': 'bf16', 'data': 'synthetic',
                      'config': {'workload': 'ce', 'shape': [rows, classes], 'l2': 'inputs larger than L2', **results},
                      'roofline': {'bound': 'hbm', 'achieved': best, 'peak': peaks['hbm_gbs'], 'unit': 'GB/s',
                                   'frac': best / peaks['hbm_gbs'], 'traffic': None, 'peak_source': peak_source}}),
          flush=True)


def layer_norm(args, device):
    """
    Layer normalisation in front of the first projection, on the C2 shape (8192 tokens, 4096 features):
    the kernels through the C ABI (fp32 in / fp32 out as PyTorch's autocast would run it, fp32 in / bf16
    out as the fused operand store, bf16 throughout), then under bf16 autocast one forward + backward of
    LayerNorm -> Linear(4096 -> 4096, gelu) as attorch_b200.LayerNormLinear, as the two layers one after
    the other, and as torch.nn.LayerNorm -> torch.nn.Linear -> gelu.  HBM-bound: forward moves
    rows * feat * (input + output element) bytes, backward rows * feat * (x + dy + dx elements).
    """
    import attorch_b200
    from attorch_b200 import _lib
    lib = _lib.load()
    peaks, peak_source = measured_peaks()
    rows, feat = 8192, 4096
    n = rows * feat
    stream = torch.cuda.current_stream().cuda_stream
    ids = {torch.float32: _lib.F32, torch.bfloat16: _lib.BF16}
    w = torch.randn(feat, device=device)
    b = torch.randn(feat, device=device)
    stats = torch.empty(2, rows, device=device)
    pgrad = torch.empty(2, feat, device=device)
    ws = torch.empty(lib.ab200_layer_norm_workspace_bytes(rows, feat), dtype=torch.uint8, device=device)
    status = torch.zeros(1, dtype=torch.int32, device=device)
    results = {}
    # Three sets of buffers per case, used in turn: 3 * (64 ... 128 MiB) per tensor is larger than L2.
    for name, xdt, ydt in (('fp32_fp32', torch.float32, torch.float32), ('fp32_bf16', torch.float32, torch.bfloat16),
                           ('bf16_bf16', torch.bfloat16, torch.bfloat16)):
        xs = [(torch.randn(rows, feat, device=device) * 2 + 0.5).to(xdt) for _ in range(3)]
        ys = [torch.empty(rows, feat, dtype=ydt, device=device) for _ in range(3)]
        dys = [torch.randn(rows, feat, device=device).to(ydt) for _ in range(3)]
        dxs = [torch.empty(rows, feat, dtype=xdt, device=device) for _ in range(3)]
        turn = [0]

        def forward():
            i = turn[0] = (turn[0] + 1) % 3
            _lib.check(lib.ab200_layer_norm_forward(xs[i].data_ptr(), w.data_ptr(), b.data_ptr(), stats[0].data_ptr(),
                                                    stats[1].data_ptr(), ys[i].data_ptr(), rows, feat, feat, feat,
                                                    ids[xdt], _lib.F32, ids[ydt], 1e-5, stream),
                       'ab200_layer_norm_forward')

        def backward():
            i = turn[0] = (turn[0] + 1) % 3
            _lib.check(lib.ab200_layer_norm_backward(dys[i].data_ptr(), xs[i].data_ptr(), stats[0].data_ptr(),
                                                     stats[1].data_ptr(), w.data_ptr(), dxs[i].data_ptr(),
                                                     pgrad[0].data_ptr(), pgrad[1].data_ptr(), rows, feat, feat, feat,
                                                     feat, ids[ydt], ids[xdt], _lib.F32, ids[xdt], ws.data_ptr(),
                                                     ws.numel(), status.data_ptr(), stream),
                       'ab200_layer_norm_backward')

        xe, ye = xs[0].element_size(), ys[0].element_size()
        for kind, fn, nbytes in (('forward', forward, n * (xe + ye)), ('backward', backward, n * (2 * xe + ye))):
            ms = event_time(fn, args.steps, max(args.warmup, 3))
            results[f'{name}_{kind}'] = {'us': round(ms * 1e3, 2), 'gbs': round(nbytes / (ms * 1e-3) / 1e9, 1)}
        del xs, ys, dys, dxs
    assert int(status.item()) == 0, 'a layer-normalisation kernel gave up on a wait'
    attorch_b200.check_status()

    # The block: LayerNorm -> Linear(gelu) under bf16 autocast, forward + backward, fp32 parameters and input.
    torch.manual_seed(0)
    norm = attorch_b200.LayerNorm(feat)
    linear = attorch_b200.Linear(feat, feat, act_func='gelu')
    fused = attorch_b200.LayerNormLinear(norm, linear)
    t_norm = torch.nn.LayerNorm(feat, device=device)
    t_linear = torch.nn.Linear(feat, feat, device=device)
    xg = (torch.randn(rows, feat, device=device) * 2 + 0.5).requires_grad_(True)
    dy = (torch.randn(rows, feat, device=device) * 0.01).bfloat16()

    def block(call, params):
        def step():
            with torch.autocast('cuda', dtype=torch.bfloat16):
                y = call(xg)
            y.backward(dy)
            xg.grad = None
            for p in params:
                p.grad = None
        return step

    ours = list(fused.parameters())
    theirs = list(t_norm.parameters()) + list(t_linear.parameters())
    for name, step in (('block_fused', block(fused, ours)),
                       ('block_two_layers', block(lambda t: linear(norm(t)), ours)),
                       ('block_torch', block(lambda t: torch.nn.functional.gelu(t_linear(t_norm(t))), theirs))):
        ms = event_time(step, args.steps, max(args.warmup, 3))
        results[name] = {'us': round(ms * 1e3, 2)}
    attorch_b200.check_status()
    best = results['fp32_bf16_forward']['gbs']
    print(json.dumps({'metric': 'layer_norm_gbs', 'value': best, 'unit': 'GB/s', 'n_gpus': 1, 'steps': args.steps,
                      'warmup': args.warmup, 'higher_is_better': True, 'dtype': 'f32', 'data': 'synthetic',
                      'config': {'workload': 'ln', 'shape': [rows, feat], 'l2': 'buffers used in turn, larger than L2',
                                 **results},
                      'roofline': {'bound': 'hbm', 'achieved': best, 'peak': peaks['hbm_gbs'], 'unit': 'GB/s',
                                   'frac': best / peaks['hbm_gbs'], 'traffic': None, 'peak_source': peak_source}}),
          flush=True)


def fused_input_gradient(args, device):
    """
    The input gradient of the C2 layer, dX[8192, 4096] = (dY (.) act'(Z))[8192, 4096] * W^T, two ways: the
    layer's path (ab200_act_backward writes dZ and the bias gradient, ab200_linear_backward_input multiplies)
    and ab200_linear_backward_input_fused, which forms dZ in the operand path (products written to tensor
    memory as the A operand) and has no bias gradient.  Reports the time of each and whether the results
    agree bit for bit.
    """
    from attorch_b200 import _lib
    lib = _lib.load()
    peaks, peak_source = measured_peaks()
    M, K, N = (args.tokens or 8192), 4096, 4096
    dy = (torch.randn(M, N, device=device) * 0.01).bfloat16()
    d = torch.rand(M, N, device=device).mul_(1.1).half()
    w = (torch.randn(K, N, device=device) / N ** 0.5).bfloat16()
    dz = torch.empty(M, N, dtype=torch.bfloat16, device=device)
    db = torch.empty(N, dtype=torch.float32, device=device)
    ws = torch.empty(max(lib.ab200_act_backward_workspace_bytes(M, N), 16), dtype=torch.uint8, device=device)
    gws_bytes = max(lib.ab200_gemm_workspace_bytes(M, K, N), 16)
    gws = torch.empty(gws_bytes, dtype=torch.uint8, device=device)
    status = torch.zeros(1, dtype=torch.int32, device=device)
    stream = torch.cuda.current_stream().cuda_stream
    flags = _lib.FLAG_FORCE_TCGEN05 | _lib.FLAG_NO_STREAMK
    results = {}
    for label, dx_dtype, dx_id in (('bf16_out', torch.bfloat16, _lib.BF16), ('fp32_out', torch.float32, _lib.F32)):
        dx_two = torch.empty(M, K, dtype=dx_dtype, device=device)
        dx_one = torch.empty(M, K, dtype=dx_dtype, device=device)

        def act_bwd():
            _lib.check(lib.ab200_act_backward(dy.data_ptr(), d.data_ptr(), dz.data_ptr(), db.data_ptr(), M, N, N, N, N,
                                              _lib.BF16, _lib.F32, _lib.ACT_SAVED_DERIVATIVE_F16, 0.0, ws.data_ptr(),
                                              ws.numel(), stream), 'ab200_act_backward')

        def product():
            _lib.check(lib.ab200_linear_backward_input(dz.data_ptr(), w.data_ptr(), dx_two.data_ptr(), M, K, N, N, 1, N, 1,
                                                       K, _lib.BF16, dx_id, gws.data_ptr(), gws_bytes,
                                                       status.data_ptr(), stream, flags), 'ab200_linear_backward_input')

        def two_kernels():
            act_bwd()
            product()

        def fused():
            _lib.check(lib.ab200_linear_backward_input_fused(dy.data_ptr(), d.data_ptr(), w.data_ptr(), dx_one.data_ptr(),
                                                             M, K, N, N, N, N, K, _lib.F16, dx_id, status.data_ptr(),
                                                             stream), 'ab200_linear_backward_input_fused')

        two_kernels()
        fused()
        torch.cuda.synchronize()
        code = int(status.item())
        assert code == 0, f'device status {code}'
        diff = (dx_one.float() - dx_two.float()).abs().max().item()
        entry = {'bit_equal': bool(torch.equal(dx_one, dx_two)), 'max_abs_diff': diff,
                 'max_abs': dx_two.float().abs().max().item()}
        for name, fn in (('act_backward_us', act_bwd), ('product_us', product), ('two_kernels_us', two_kernels),
                         ('fused_us', fused)):
            entry[name] = round(event_time(fn, args.steps, max(args.warmup, 3)) * 1e3, 2)
        entry['fused_tflops'] = round(2.0 * M * K * N / (entry['fused_us'] * 1e-6) / 1e12, 1)
        results[label] = entry
        del dx_two, dx_one
    assert int(status.item()) == 0, 'a kernel gave up on a wait'
    best = results['bf16_out']['fused_tflops']
    print(json.dumps({'metric': 'fused_input_gradient_tflops', 'value': best, 'unit': 'TFLOP/s', 'n_gpus': 1,
                      'steps': args.steps, 'warmup': args.warmup, 'higher_is_better': True, 'dtype': 'bf16',
                      'data': 'synthetic', 'config': {'workload': 'dxfused', 'shape': [M, K, N], **results},
                      'roofline': {'bound': 'tensor', 'achieved': best, 'peak': peaks['bf16_tflops'], 'unit': 'TFLOP/s',
                                   'frac': best / peaks['bf16_tflops'], 'traffic': None, 'peak_source': peak_source}}),
          flush=True)


class Comm:
    """Rank, world size and the two collectives the timing protocol needs."""
    def __init__(self, device, world_size, rank):
        self.device, self.world_size, self.rank = device, world_size, rank

    def barrier(self):
        if self.world_size > 1:
            import torch.distributed as dist
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(self, value):
        if self.world_size == 1:
            return value
        import torch.distributed as dist
        t = torch.tensor([value], dtype=torch.float64, device=self.device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())


class StepRunner:
    """
    One workload on one rank: the layers, their gradient buckets, a resident batch, and a step
    function under one of these schedules.
      graph          N = 1: the whole step is one captured CUDA graph (eager with --no-graph).
      graph_split    N > 1, one layer: graph 1 = casts, forward, activation backward, dW; then the
                     all-reduce of the bucket starts on a side stream; graph 2 = dX on the SMs NCCL's
                     kernel leaves free (as many as NCCL_MAX_CTAS allows it).  NCCL itself is not
                     captured.  (Launching only the first rows of dX beside the exchange and the rest on
                     all SMs afterwards measured slower at 2 GPUs: 0.76-0.79 ms against 0.744 ms.)
      eager_overlap  N > 1, any model: eager launches, each layer's all-reduce issued from inside
                     backward per block of dW, overlapping the rest of backward.
      graph_serial   N > 1: one graph of the local step, then one all-reduce (no overlap).
      graph_overlap  N > 1 with the library's own all-reduce kernel (NVLink multicast): like
                     eager_overlap, but the kernel is capturable, so the whole step - exchange on its
                     side stream included - is one CUDA graph again.  The default where multicast works.
    `local_only` builds the same step without any exchange although other ranks exist.
    """
    def __init__(self, name, spec, comm, lib, tokens=None, schedule=None, no_graph=False, local_only=False):
        import attorch_b200
        from attorch_b200.dp import GradientBuckets
        self.ab = attorch_b200
        self.name, self.spec, self.comm, self.lib = name, spec, comm, lib
        device, world_size, rank = comm.device, comm.world_size, comm.rank
        self.device = device
        self.distributed = world_size > 1 and not local_only
        self.tokens = tokens or spec['tokens_per_gpu'] or spec['global_tokens'] // (world_size if self.distributed else 1)
        torch.manual_seed(0)
        self.layers = [attorch_b200.Linear(k, n, bias=bias, act_func=act, device=device, dtype=spec['param_dtype'])
                       for (k, n, act, bias) in spec['layers']]
        grad_dtype = {'bf16': torch.bfloat16, 'fp16': torch.float16, 'fp32': torch.float32, '': None}[
            os.environ.get('AB200_GRAD_DTYPE', '')]
        if grad_dtype is None and self.distributed and spec['autocast'] is not None:
            grad_dtype = spec['autocast']      # exchange in the autocast dtype, widen into the fp32 .grad
        if not self.distributed:
            schedule = 'eager' if no_graph else 'graph'
        elif schedule is None:
            schedule = os.environ.get('AB200_SCHEDULE')
        transport = os.environ.get('AB200_TRANSPORT', 'auto') if self.distributed else 'nccl'
        self.buckets = None
        if self.distributed and transport != 'nccl' and schedule in (None, 'graph_overlap'):
            # The library's own all-reduce, the whole bucket of a layer in one call.  4 CTAs measured
            # best for workload c2 at 2, 4 and 8 GPUs (8 GPUs: 0.735 / 0.740 / 0.754 ms with 4 / 8 / 16).
            ctas = int(os.environ.get('AB200_COMM_CTAS', '4'))
            buckets = GradientBuckets(self.layers, overlap=True, dw_chunks=int(os.environ.get('AB200_DW_CHUNKS', '1')),
                                      grad_dtype=grad_dtype, transport=transport, comm_ctas=ctas)
            if buckets.transport == 'multimem':
                self.buckets, schedule, self.comm_sms = buckets, 'graph_overlap', ctas
        if self.buckets is None:
            if self.distributed and schedule in (None, 'graph_overlap'):
                schedule = 'graph_split' if len(self.layers) == 1 else 'eager_overlap'
            self.comm_sms = int(os.environ.get('AB200_COMM_SMS', '32')) if self.distributed else 0
            self.buckets = GradientBuckets(
                self.layers, overlap=(schedule == 'eager_overlap'), comm_sms=self.comm_sms,
                dw_chunks=int(os.environ.get('AB200_DW_CHUNKS', '2')),
                defer_first_input_grad=(schedule == 'graph_split'),
                grad_dtype=grad_dtype if self.distributed else None, exchange=self.distributed)
        self.schedule = schedule
        self.k_in, self.n_out = spec['layers'][0][0], spec['layers'][-1][1]
        gen = torch.Generator(device=device).manual_seed(1 + rank)
        self.x = torch.randn(self.tokens, self.k_in, device=device, generator=gen).to(spec['input_dtype'])
        self.x.requires_grad_(True)
        out_dtype = spec['autocast'] or spec['param_dtype']
        self.dy = (torch.randn(self.tokens, self.n_out, device=device, generator=gen) * 0.01).to(out_dtype)
        self.graphs = None
        self.output = None

    # -- pieces of a step
    def compute(self, x):
        self.buckets.zero_grad()
        x.grad = None
        spec = self.spec
        with torch.autocast('cuda', dtype=spec['autocast'] or torch.bfloat16, enabled=spec['autocast'] is not None):
            h = x
            for layer in self.layers:
                h = layer(h)
        self.output = h.detach()      # not h itself: that would keep this step's autograd graph alive
        h.backward(self.dy)

    def step(self, x):
        """One eager step (every schedule can run eagerly: warm-up, launch counting, end-to-end loop)."""
        self.compute(x)
        if self.schedule == 'graph_split':
            self.buckets.start_exchange()
            self.buckets.run_deferred(reserve_sms=self.comm_sms)
        self.buckets.finish()

    def time_exchange(self):
        """The exchange alone and the deferred dX alone (ms, max over ranks): how much there is to hide, and where."""
        if self.schedule != 'graph_split':
            return None
        for _ in range(2):
            self.step(self.x)
        torch.cuda.synchronize()

        def exchange():
            self.buckets.start_exchange()
            self.buckets.finish()

        self.compute(self.x)          # leaves the dX launcher registered

        def product():
            self.buckets.run_deferred(keep=True)

        self.comm.barrier()
        exchange_ms = self.comm.max_over_ranks(event_time(exchange, 5, 2))
        product_ms = self.comm.max_over_ranks(event_time(product, 5, 2))
        self.buckets.run_deferred()
        return {'exchange_alone_ms': exchange_ms, 'deferred_dx_alone_ms': product_ms}

    def capture(self):
        """Captures the local pieces of a step as CUDA graphs; returns False if capture is not used."""
        if self.schedule in ('eager', 'eager_overlap'):
            return False
        side = torch.cuda.Stream(self.device)
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for _ in range(3):
                self.step(self.x)
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        graphs = [torch.cuda.CUDAGraph()]
        with torch.cuda.graph(graphs[0]):
            if self.schedule == 'graph_overlap':
                self.step(self.x)       # the exchange (on its side stream) is part of the graph
            else:
                self.compute(self.x)
        if self.schedule == 'graph_split':
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, pool=graphs[0].pool()):
                self.buckets.run_deferred(reserve_sms=self.comm_sms)
            graphs.append(graph)
        self.graphs = graphs
        self.run()
        torch.cuda.synchronize()
        self.ab.check_status()
        return True

    def run(self):
        if self.graphs is None:
            self.step(self.x)
            return
        self.graphs[0].replay()
        if self.schedule == 'graph_overlap':
            return
        if self.schedule == 'graph_split':
            self.buckets.start_exchange()
            for graph in self.graphs[1:]:
                graph.replay()
        self.buckets.finish()

    def timed(self, steps, sample_clocks_on=-1):
        """Times `steps` runs: (ms per step as the max over ranks, host ms per step, clock summary)."""
        for _ in range(3):
            self.run()
        self.comm.barrier()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        with ClockSampler(sample_clocks_on) as clocks:
            self.comm.barrier()
            start.record()
            host_t0 = time.perf_counter()
            for _ in range(steps):
                self.run()
            host_ms = (time.perf_counter() - host_t0) * 1e3 / steps
            stop.record()
            self.comm.barrier()
        ms = self.comm.max_over_ranks(start.elapsed_time(stop)) / steps
        self.ab.check_status()
        return ms, host_ms, clocks.summary()

    def launches_per_step(self):
        before = self.lib.ab200_launch_count()
        self.step(self.x)
        torch.cuda.synchronize()
        return self.lib.ab200_launch_count() - before

    def collective_bytes(self):
        return self.buckets.flat.numel() * self.buckets.flat.element_size()


def torch_gpu_baseline(spec, tokens, device, steps, warmup):
    """
    The same step in PyTorch on the same GPU: torch.nn.Linear + F.gelu under bf16 autocast with fp32
    parameters and input, forward + backward (cuBLAS GEMMs, PyTorch's cast / activation / reduction
    kernels), and the three bare matmuls of the step alone.  Same CUDA-event protocol.
    """
    import torch.nn.functional as F
    k, n, act, bias = spec['layers'][0]
    layer = torch.nn.Linear(k, n, bias=bias, device=device, dtype=spec['param_dtype'])
    x = torch.randn(tokens, k, device=device, dtype=spec['input_dtype'], requires_grad=True)
    dy = (torch.randn(tokens, n, device=device) * 0.01).to(spec['autocast'] or spec['param_dtype'])
    act_fn = {None: (lambda t: t), 'gelu': F.gelu, 'silu': F.silu, 'relu': F.relu}[act]

    def step():
        x.grad = None
        layer.zero_grad(set_to_none=True)
        with torch.autocast('cuda', dtype=spec['autocast'] or torch.bfloat16, enabled=spec['autocast'] is not None):
            y = act_fn(layer(x))
        y.backward(dy)

    eager_ms = event_time(step, steps, warmup)
    graph_ms = None
    try:
        side = torch.cuda.Stream(device)
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for _ in range(3):
                step()
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            step()
        graph_ms = event_time(graph.replay, steps, warmup)
    except Exception as error:
        print(f'torch baseline: graph capture failed ({error})', file=sys.stderr)
        torch.cuda.synchronize()
    op = spec['autocast'] or spec['param_dtype']
    xb = torch.randn(tokens, k, device=device).to(op)
    wb = torch.randn(n, k, device=device).to(op)       # torch.nn.Linear layout [out, in]
    dz = torch.randn(tokens, n, device=device).to(op)
    yb = torch.empty(tokens, n, device=device, dtype=op)
    dxb = torch.empty(tokens, k, device=device, dtype=op)
    dwb = torch.empty(n, k, device=device, dtype=op)
    matmuls = {'forward': event_time(lambda: torch.matmul(xb, wb.t(), out=yb), steps, warmup),
               'dX': event_time(lambda: torch.matmul(dz, wb, out=dxb), steps, warmup),
               'dW': event_time(lambda: torch.matmul(dz.t(), xb, out=dwb), steps, warmup)}
    flops = flops_per_step(spec, tokens)
    best = min(v for v in (eager_ms, graph_ms) if v is not None)
    return {'what': 'torch.nn.Linear + F.gelu forward + backward under bf16 autocast, fp32 parameters and '
                    'input, same GPU, same protocol',
            'ms_per_step_eager': eager_ms, 'ms_per_step_graph': graph_ms, 'tflops': flops / (best * 1e-3) / 1e12,
            'bare_matmul_ms': matmuls, 'bare_matmul_sum_ms': sum(matmuls.values()),
            'bare_matmul_tflops': flops / (sum(matmuls.values()) * 1e-3) / 1e12}


def dp_parity(comm):
    """
    Data-parallel gradients against full-batch gradients, on the GPUs, outside any timed region: every
    rank runs one step on its shard of a small batch (bf16 autocast, fp32 parameters, upstream gradient
    N(0, 1) * 0.01 as in workload c2; fp32 and bf16 exchange); the shards are all-gathered and every rank computes the full-batch dW / db with the same
    kernels; the all-reduced ``.grad`` must equal them within rtol = atol = 1e-2.
    """
    import torch.distributed as dist

    import attorch_b200
    from attorch_b200.dp import GradientBuckets
    device, world_size, rank = comm.device, comm.world_size, comm.rank
    rows, k, n = 512, 1024, 768
    report = {'shape': [rows * world_size, k, n], 'rtol_atol': 1e-2}
    cases = [(None, 'nccl', 'fp32_exchange'), (torch.bfloat16, 'nccl', 'bf16_exchange')]
    if os.environ.get('AB200_TRANSPORT', 'auto') != 'nccl':
        cases.append((torch.bfloat16, 'auto', 'bf16_exchange_own_kernel'))
    for exchange_dtype, transport, tag in cases:
        torch.manual_seed(3)
        layer = attorch_b200.Linear(k, n, bias=True, act_func='gelu', device=device, dtype=torch.float32)
        full = attorch_b200.Linear(k, n, bias=True, act_func='gelu', device=device, dtype=torch.float32)
        full.load_state_dict(layer.state_dict())
        buckets = GradientBuckets([layer], overlap=True, comm_sms=32, dw_chunks=2, grad_dtype=exchange_dtype,
                                  transport=transport)
        gen = torch.Generator(device=device).manual_seed(100 + rank)
        x = torch.randn(rows, k, device=device, generator=gen)
        dy = (torch.randn(rows, n, device=device, generator=gen) * 0.01).bfloat16()
        xg = x.clone().requires_grad_(True)
        with torch.autocast('cuda', dtype=torch.bfloat16):
            y = layer(xg)
        y.backward(dy)
        buckets.finish()
        xs = [torch.empty_like(x) for _ in range(world_size)]
        dys = [torch.empty_like(dy) for _ in range(world_size)]
        dist.all_gather(xs, x)
        dist.all_gather(dys, dy)
        xf = torch.cat(xs).requires_grad_(True)
        with torch.autocast('cuda', dtype=torch.bfloat16):
            yf = full(xf)
        yf.backward(torch.cat(dys))
        torch.cuda.synchronize()
        attorch_b200.check_status()
        ok, worst = True, 0.0
        for got, want in ((layer.weight.grad, full.weight.grad), (layer.bias.grad, full.bias.grad)):
            err = (got.float() - want.float()).abs()
            bound = 1e-2 + 1e-2 * want.float().abs()
            worst = max(worst, float((err / bound).max().item()))
            ok = ok and bool((err <= bound).all().item())
        # The shard's own dX must equal the rows of the full-batch dX it owns.
        own = xf.grad[rank * rows:(rank + 1) * rows]
        ok = ok and bool(torch.allclose(xg.grad, own, rtol=1e-2, atol=1e-2))
        flag = torch.tensor([1 if ok else 0], device=device)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        report[tag] = {'ok': bool(flag.item() == 1), 'worst_error_over_bound_rank0': worst,
                       'transport': buckets.transport}
        del buckets, layer, full
    report['ok'] = all(report[t]['ok'] for (_, _, t) in cases)
    return report


def all_reduce_times(comm):
    """
    All-reduce of 32 / 64 / 256 MiB on otherwise idle GPUs, NCCL and (where NVLink multicast works) the
    library's own kernel on 8 CTAs: ms and bus bandwidth (max over ranks).
    """
    import torch.distributed as dist

    from attorch_b200.dp import _MultimemBucket
    out = []
    n = comm.world_size
    for mib, dtype in ((32, torch.bfloat16), (64, torch.float32), (256, torch.bfloat16)):
        elt = torch.empty(0, dtype=dtype).element_size()
        numel = mib * 1024 * 1024 // elt
        nbytes = numel * elt
        buf = torch.zeros(numel, dtype=dtype, device=comm.device)
        comm.barrier()
        ms = comm.max_over_ranks(event_time(lambda: dist.all_reduce(buf), 10, 3))
        row = {'mib': mib, 'dtype': DTYPE_NAMES[dtype], 'nccl_ms': ms,
               'nccl_busbw_gbs': nbytes * 2.0 * (n - 1) / n / (ms * 1e-3) / 1e9}
        del buf
        if os.environ.get('AB200_TRANSPORT', 'auto') != 'nccl':
            try:
                bucket = _MultimemBucket(numel, dtype, comm.device, None, int(os.environ.get('AB200_COMM_CTAS', '8')))
                comm.barrier()
                ms = comm.max_over_ranks(event_time(lambda: bucket.all_reduce(0, numel), 10, 3))
                row.update({'own_kernel_ms': ms, 'own_kernel_ctas': bucket.ctas,
                            'own_kernel_busbw_gbs': nbytes * 2.0 * (n - 1) / n / (ms * 1e-3) / 1e9})
                del bucket
            except Exception as error:
                row['own_kernel'] = f'unavailable: {error}'
        out.append(row)
    return out


def end_to_end(runner, comm, steps):
    """
    The same step fed from host memory: every step copies its input from pinned host memory (next
    step's copy overlapping this step's compute on a side stream) and reads the step's output and the
    last layer's bias gradient back into pinned host memory (on another side stream, overlapping the
    next step).  Returns (ms per step, host-to-device bytes, device-to-host bytes per step).
    """
    spec, device = runner.spec, runner.device
    host_x = [torch.randn(runner.tokens, runner.k_in).to(spec['input_dtype']).pin_memory() for _ in range(2)]
    dev_x = [torch.empty_like(runner.x).requires_grad_(True) for _ in range(2)]
    out_dtype = spec['autocast'] or spec['param_dtype']
    host_y = torch.empty(runner.tokens, runner.n_out, dtype=out_dtype).pin_memory()
    last = runner.layers[-1]
    small = last.bias if last.bias is not None else last.weight[0]
    host_small = torch.empty(small.shape, dtype=small.dtype).pin_memory()
    copy_stream = torch.cuda.Stream(device)
    back_stream = torch.cuda.Stream(device)
    copied = [torch.cuda.Event() for _ in range(2)]
    consumed = [torch.cuda.Event() for _ in range(2)]
    produced = torch.cuda.Event()
    read_back = torch.cuda.Event()

    def loop(n_steps):
        compute = torch.cuda.current_stream()
        with torch.cuda.stream(copy_stream):
            dev_x[0].data.copy_(host_x[0], non_blocking=True)
            copied[0].record(copy_stream)
        for i in range(n_steps):
            cur, nxt = i % 2, (i + 1) % 2
            if i + 1 < n_steps:
                with torch.cuda.stream(copy_stream):
                    if i >= 1:
                        copy_stream.wait_event(consumed[nxt])
                    dev_x[nxt].data.copy_(host_x[nxt], non_blocking=True)
                    copied[nxt].record(copy_stream)
            compute.wait_event(copied[cur])
            runner.step(dev_x[cur])
            consumed[cur].record(compute)
            produced.record(compute)
            output = runner.output.view(runner.tokens, runner.n_out)
            grad = last.bias.grad if last.bias is not None else last.weight.grad[0]
            with torch.cuda.stream(back_stream):
                back_stream.wait_event(produced)
                host_y.copy_(output, non_blocking=True)
                host_small.copy_(grad, non_blocking=True)
                read_back.record(back_stream)
            # Keeps the output's memory from being handed to the next step before it has been read.
            output.record_stream(back_stream)
            grad.record_stream(back_stream)
        compute.wait_event(read_back)
        compute.synchronize()

    loop(3)
    comm.barrier()
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0.record()
    loop(steps)
    t1.record()
    comm.barrier()
    ms = comm.max_over_ranks(t0.elapsed_time(t1)) / steps
    h2d = host_x[0].numel() * host_x[0].element_size()
    d2h = host_y.numel() * host_y.element_size() + host_small.numel() * host_small.element_size()
    return ms, h2d, d2h


def main():
    parser = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawTextHelpFormatter)
    parser.add_argument('--gpus', type=int, default=1)
    parser.add_argument('--steps', type=int, default=200)
    parser.add_argument('--warmup', type=int, default=10)
    parser.add_argument('--workload', choices=sorted(WORKLOADS) + ['c4', 'act', 'ce', 'ln', 'dxfused'], default='c2')
    parser.add_argument('--only', default=None,
                        help='workload act: time just this entry (e.g. kernel_forward, glu_backward)')
    parser.add_argument('--impl', choices=['b200', 'reference'], default='b200')
    parser.add_argument('--no-cpu-baseline', action='store_true')
    parser.add_argument('--no-extras', action='store_true',
                        help='only the timed workload: no sub-records for the other workloads and baselines')
    parser.add_argument('--no-graph', action='store_true',
                        help='launch every step eagerly instead of replaying captured CUDA graphs')
    parser.add_argument('--kernel-only', choices=['fwd', 'dx', 'dw', 'act_bwd'], default=None,
                        help='launch only this kernel of the first layer (for ncu captures)')
    parser.add_argument('--tokens', type=int, default=None,
                        help='override the tokens per GPU (profiling of reduced cases)')
    args = parser.parse_args()
    args.warmup = max(args.warmup, 3)
    if args.workload in ('c4', 'act', 'ce', 'ln', 'dxfused'):
        if args.impl == 'reference':
            print(json.dumps({'impl': 'reference', 'unavailable': f'{args.workload} has no CPU arm; use c2'}))
            return
        from attorch_b200 import _lib
        torch.cuda.set_device(0)
        if args.workload == 'c4':
            print(json.dumps(skinny_forward(args.steps, args.warmup, torch.device('cuda', 0), _lib.load())), flush=True)
        elif args.workload == 'ce':
            cross_entropy_loss(args, torch.device('cuda', 0))
        elif args.workload == 'ln':
            layer_norm(args, torch.device('cuda', 0))
        elif args.workload == 'dxfused':
            fused_input_gradient(args, torch.device('cuda', 0))
        else:
            activation_layer(args, torch.device('cuda', 0))
        return
    spec = WORKLOADS[args.workload]

    world_size = int(os.environ.get('WORLD_SIZE', '1'))
    rank = int(os.environ.get('RANK', '0'))
    local_rank = int(os.environ.get('LOCAL_RANK', '0'))
    if args.impl == 'reference':
        run_reference(args, spec, max(world_size, args.gpus), rank)
        return

    import torch.distributed as dist

    import attorch_b200
    from attorch_b200 import _lib

    if not torch.cuda.is_available():
        raise SystemExit('bench.py needs a CUDA device: the layer has no CPU fallback')
    lib = _lib.load()
    torch.cuda.set_device(local_rank)
    device = torch.device('cuda', local_rank)
    log = None
    if world_size > 1:
        os.environ.setdefault('MASTER_ADDR', '127.0.0.1')
        # The GEMM that runs beside the exchange leaves exactly the SMs NCCL's kernel occupies.
        os.environ.setdefault('NCCL_MAX_CTAS', os.environ.get('AB200_COMM_SMS', '32'))
        log = CollectiveLog()
        dist.init_process_group('nccl', device_id=device)
    comm = Comm(device, world_size, rank)

    if args.kernel_only:
        tokens = args.tokens or spec['tokens_per_gpu'] or spec['global_tokens'] // world_size
        kernel_only(args, spec, tokens, device, lib)
        return

    # ---------------------------------------------------------------- device-resident timing
    runner = StepRunner(args.workload, spec, comm, lib, tokens=args.tokens, no_graph=args.no_graph)
    tokens, total_tokens = runner.tokens, runner.tokens * world_size
    for _ in range(args.warmup):
        runner.step(runner.x)
    comm.barrier()
    attorch_b200.check_status()
    calibration = runner.time_exchange()
    graphed = False
    try:
        graphed = runner.capture()
    except Exception as error:  # capture unsupported here: time the eager loop instead
        print(f'CUDA graph capture failed, timing eager launches: {error}', file=sys.stderr)
        runner.graphs = None
        torch.cuda.synchronize()
    ms_per_step, host_ms_per_step, clocks = runner.timed(args.steps, local_rank if rank == 0 else -1)
    launches = runner.launches_per_step() * args.steps
    step_flops = flops_per_step(spec, tokens)
    value = step_flops * world_size / (ms_per_step * 1e-3) / 1e12
    collective_bytes = runner.collective_bytes()
    schedule, comm_sms = runner.schedule, runner.comm_sms
    exchange_dtype, param_dtype, widened = runner.buckets.grad_dtype, runner.buckets.dtype, runner.buckets.widen
    transport = runner.buckets.transport

    # The same local computation without any exchange (at N = 1 this is the step itself): what is
    # left of a data-parallel step after subtracting it is communication that was not hidden.
    local_ms = ms_per_step
    if world_size > 1:
        solo = StepRunner(args.workload, spec, comm, lib, tokens=tokens, local_only=True)
        for _ in range(3):
            solo.step(solo.x)
        solo.capture()
        local_ms, _, _ = solo.timed(args.steps)
        del solo
        torch.cuda.empty_cache()

    # ---------------------------------------------------------------- end to end with host buffers
    e2e_steps = max(10, min(args.steps, 40))
    e2e_ms, h2d_bytes, d2h_bytes = end_to_end(runner, comm, e2e_steps)
    e2e_value = step_flops * world_size / (e2e_ms * 1e-3) / 1e12
    attorch_b200.check_status()
    del runner
    torch.cuda.empty_cache()

    # ---------------------------------------------------------------- roofline of the dominant kernel
    # The tcgen05 GEMM, launched through the C ABI exactly as the layer launches it (forward of the
    # first layer: X[M, K] * W[K, N] with bias, gelu and the saved-derivative store), event-timed on
    # the launching stream.
    peaks, peak_source = measured_peaks()
    k0, n0 = spec['layers'][0][0], spec['layers'][0][1]
    launch_fwd, _, _ = kernel_launcher(spec, tokens, device, lib, 'fwd')
    kernel_ms = event_time(launch_fwd, 30, 5)
    del launch_fwd
    achieved = 2.0 * tokens * k0 * n0 / (kernel_ms * 1e-3) / 1e12
    roofline = {'bound': 'tensor', 'achieved': achieved, 'peak': peaks['bf16_tflops'], 'unit': 'TFLOP/s',
                'frac': achieved / peaks['bf16_tflops'],
                'traffic': profiled_dram_bytes() if (args.workload == 'c2' and tokens == 8192) else None,
                'traffic_source': 'ncu dram__bytes_read.sum + dram__bytes_write.sum per launch, from the committed '
                                  'summary profiles/c2_kernel_fwd.md',
                'algorithmic_bytes': 2.0 * (tokens * k0 + k0 * n0 + 2 * tokens * n0),
                'kernel': 'gemm_tcgen05_kernel (forward: bias + gelu + saved-derivative epilogue)',
                'kernel_ms': kernel_ms, 'peak_source': f'{peak_source} (cuBLAS bf16 burst)',
                'frac_of_nominal_2250': achieved / 2250.0}
    kernels = {}
    if not args.no_extras:
        for which in ('dx', 'dw', 'act_bwd'):
            launch, work, unit = kernel_launcher(spec, tokens, device, lib, which)
            ms = event_time(launch, 20, 3)
            kernels[which] = {'ms': ms, ('tflops' if unit == 'flops' else 'gbs'):
                              work / (ms * 1e-3) / (1e12 if unit == 'flops' else 1e9)}
            del launch
            torch.cuda.empty_cache()

    # ---------------------------------------------------------------- sub-records
    extras = {}
    collective = {'kind': 'none'}
    if world_size > 1:
        choice = log.all_reduce_choice(collective_bytes)
        collective = {
            'kind': 'all-reduce (SUM) of dW/db', 'transport': transport, 'schedule': schedule,
            'dtype': DTYPE_NAMES[exchange_dtype], 'bytes': collective_bytes,
            'widened_to': DTYPE_NAMES[param_dtype] if widened else None,
            'sms_left_free_beside_it': comm_sms, **(calibration or {})}
        if transport == 'multimem':
            collective.update({
                'algorithm': 'own kernel: multimem.ld_reduce + multimem.st through NVSwitch (NVLink multicast), '
                             'two cross-rank barriers', 'ctas': comm_sms})
        else:
            collective.update({
                'algorithm': 'NCCL ' + (choice[0] if choice else '(algorithm not logged)'),
                'protocol': choice[1] if choice else None, 'channels': choice[2] if choice else None,
                'nccl_max_ctas': os.environ.get('NCCL_MAX_CTAS')})
    if not args.no_extras:
        if world_size > 1:
            extras['dp_parity'] = dp_parity(comm)
            extras['collectives'] = all_reduce_times(comm)
            torch.cuda.empty_cache()
        if args.workload == 'c2':
            # Two layers 8192 -> 8192, global batch 65536 split by rows (strong scaling).
            c5_spec = WORKLOADS['c5']
            c5 = StepRunner('c5', c5_spec, comm, lib)
            for _ in range(3):
                c5.step(c5.x)
            c5_graphed = False
            try:
                c5_graphed = c5.capture()
            except Exception as error:
                print(f'c5: CUDA graph capture failed ({error})', file=sys.stderr)
                c5.graphs = None
                torch.cuda.synchronize()
            c5_steps = max(5, min(args.steps, 10))
            c5_ms, _, _ = c5.timed(c5_steps)
            c5_flops = flops_per_step(c5_spec, c5_spec['global_tokens'])
            record = {'ms_per_step': c5_ms, 'tflops_total': c5_flops / (c5_ms * 1e-3) / 1e12,
                      'tflops_per_gpu': c5_flops / world_size / (c5_ms * 1e-3) / 1e12,
                      'frac_of_nominal_2250_per_gpu': c5_flops / world_size / (c5_ms * 1e-3) / 1e12 / 2250.0,
                      'tokens_per_gpu': c5.tokens, 'steps': c5_steps, 'schedule': c5.schedule,
                      'cuda_graph': c5_graphed,
                      'collective_bytes': c5.collective_bytes() if world_size > 1 else 0,
                      'scaling': 'strong'}
            del c5
            torch.cuda.empty_cache()
            if world_size > 1:
                # The whole 65536-token batch on one GPU (every rank runs it alone, no exchange).
                one = StepRunner('c5', c5_spec, comm, lib, tokens=c5_spec['global_tokens'], local_only=True)
                for _ in range(2):
                    one.step(one.x)
                one.capture()
                one_ms, _, _ = one.timed(3)
                del one
                torch.cuda.empty_cache()
                record['n1_ms_per_step_same_box'] = one_ms
                record['strong_scaling_efficiency'] = one_ms / (world_size * c5_ms)
            extras['c5'] = record
        if world_size == 1 and args.workload == 'c2':
            base = torch_gpu_baseline(spec, tokens, device, args.steps, args.warmup)
            base['this_library_over_torch'] = value / base['tflops']
            extras['torch_gpu_baseline'] = base
            torch.cuda.empty_cache()
            c3_spec = WORKLOADS['c3']
            c3 = StepRunner('c3', c3_spec, comm, lib)
            for _ in range(3):
                c3.step(c3.x)
            c3.capture()
            c3_ms, _, _ = c3.timed(max(5, min(args.steps, 10)))
            c3_flops = flops_per_step(c3_spec, c3.tokens)
            extras['c3'] = {'ms_per_step': c3_ms, 'tflops': c3_flops / (c3_ms * 1e-3) / 1e12,
                            'frac_of_nominal_2250': c3_flops / (c3_ms * 1e-3) / 1e12 / 2250.0,
                            'tokens': c3.tokens, 'layers': ['4096->14336 silu', '14336->4096']}
            del c3
            torch.cuda.empty_cache()
            # A pause first: c4 is a burst of 80 us kernels bound by HBM, and measured right after the
            # seconds of sustained GEMMs above it runs at the clocks the power limiter left behind
            # (5.3 TB/s instead of the 6.3 TB/s it reaches from idle).
            torch.cuda.synchronize()
            time.sleep(1.5)
            c4 = skinny_forward(30, 5, device, lib)
            extras['c4'] = {'unit': 'GB/s of weight read, against 8000 nominal and the measured copy bandwidth',
                            'rows': c4['config']['rows']}
            torch.cuda.empty_cache()

    comm_log_tail = ''
    if world_size > 1:
        dist.barrier()
        dist.destroy_process_group()
        comm_log_tail = log.close(echo=(rank == 0))
    if rank != 0:
        return

    line = {
        'metric': 'linear_fwd_bwd_tflops', 'value': value, 'unit': 'TFLOP/s', 'n_gpus': world_size,
        'steps': args.steps, 'warmup': args.warmup, 'ms_per_step': ms_per_step,
        'host_enqueue_ms_per_step': host_ms_per_step,
        'local_ms_per_step_without_exchange': local_ms,
        'exposed_communication_ms_per_step': max(0.0, ms_per_step - local_ms),
        'higher_is_better': True, 'scaling': spec['scaling'], 'vs_baseline': None,
        'dtype': 'bf16', 'data': 'synthetic',
        'config': {'workload': args.workload,
                   'layers': [f'{k}->{n} act={act} bias={bias}' for (k, n, act, bias) in spec['layers']],
                   'tokens_per_gpu': tokens, 'global_tokens': total_tokens,
                   'params': str(spec['param_dtype']).replace('torch.', ''),
                   'input': str(spec['input_dtype']).replace('torch.', ''),
                   'autocast': str(spec['autocast']).replace('torch.', ''),
                   'parallelism': f'dp{world_size}',
                   'collective': collective,
                   'cuda_graph': graphed,
                   'l2': 'per-step working set (operands, activations, gradients) exceeds the 126 MB L2; no flush',
                   'tflops_per_gpu': value / world_size,
                   'frac_of_nominal_2250_per_gpu': value / world_size / 2250.0},
        'clocks': clocks,
        'e2e': {'value': e2e_value, 'unit': 'TFLOP/s', 'ms_per_step': e2e_ms,
                'h2d_bytes_per_step': h2d_bytes, 'd2h_bytes_per_step': d2h_bytes,
                'host_link_gbs_per_gpu': (h2d_bytes + d2h_bytes) / (e2e_ms * 1e-3) / 1e9,
                'bound': 'host-device copies (PCIe and host memory, shared by the ranks of a box)',
                'read_back': 'the step\'s output and the last layer\'s bias gradient'},
        'gpu_launches': int(launches),
        'roofline': roofline,
        'kernels': kernels,
        **extras,
    }
    if world_size > 1:
        line['comm_log_tail'] = comm_log_tail
    if world_size == 1 and not args.no_cpu_baseline:
        seconds, threads = cpu_arm(spec, tokens, steps=5, warmup=1)
        line['cpu_baseline'] = {
            'value': flops_per_step(spec, tokens) / seconds / 1e12, 'unit': 'TFLOP/s', 'cores': threads,
            'kind': 'port',
            'sample': f'all {tokens} rows of the batch per step, 5 steps, torch.nn.Linear + activation '
                      f'fwd+bwd in fp32 on {threads} host threads'}
    print(json.dumps(line), flush=True)


if __name__ == '__main__':
    main()
