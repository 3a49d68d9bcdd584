"""
Benchmark of the fused linear layer (forward + backward) on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload c2|c3|c4|c5|act] [--impl reference]

For N > 1 launch one rank per GPU with torchrun (RANK / LOCAL_RANK / WORLD_SIZE / MASTER_* from the
environment).  Rank 0 prints one JSON line.

Workloads (synthetic, seeded; shapes of BASELINE.json's configs):
  c2  attorch.Linear 4096 -> 4096, bias, gelu, under bf16 autocast with fp32 parameters and fp32
      input; 8192 tokens per GPU (weak scaling: the global batch is 8192 * N); forward + backward
      (dX, dW, db); with N > 1 the fp32 dW / db are SUM-all-reduced every step, overlapped with dX.
  c5  two layers 8192 -> 8192 (gelu + bias, then bias), bf16 parameters, global batch 65536 tokens
      split over the N GPUs (strong scaling), same all-reduce.
  c3  transformer MLP pair 4096 -> 14336 (silu) -> 4096, no biases, bf16, 16384 tokens per GPU.
  c4  skinny forward only, fp16, 8192 -> 28672, M in {1, 8, 32, 128}: prints weight-read GB/s.
  act standalone activation layer (GELU, drop_p = 0.1, bf16, 32768 x 4096 elements) and gated linear
      unit (silu, bf16, 16384 x 2*14336): GB/s.

One "step" is one forward + backward of the workload on one batch.  ``value`` is the whole-job
TFLOP/s at 6 * M * K * N floating-point operations per layer and step with the inputs resident in
HBM; ``e2e`` is the same through the same module with the step's input copied from pinned host
memory and the bias gradient read back every step (copies double-buffered on a side stream).
``--impl reference`` times the CPU computation the reference's tests compare against
(torch.nn.Linear + activation, all host cores) on a bounded sample of the same workload.
"""

import argparse
import json
import os
import statistics
import sys
import threading
import time
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

PEAK_FALLBACK = {'hbm_gbs': 6650.0, 'bf16_tflops': 1590.0, 'bf16_tflops_sustained': 1400.0}

# DRAM bytes per launch of the dominant kernel (forward GEMM of c2) from the ncu capture summarised
# in profiles/c2_kernel_fwd.md (algorithmic bytes: 224 MiB = 234.9e6).
NCU_DRAM_BYTES_PER_LAUNCH = 255.3e6   # profiles/c2_kernel_fwd.md: 150.6 MB read + 104.7 MB written

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
# Workload c4 (BASELINE.json config 4) is forward only and HBM-bound: see skinny_forward().


def measured_peaks():
    path = ROOT / 'MEASURED_PEAKS.json'
    if path.exists():
        data = json.loads(path.read_text())
        return {k: float(data[k]) for k in PEAK_FALLBACK}, 'measured'
    return dict(PEAK_FALLBACK), 'fallback'


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


def flops_per_step(spec, tokens):
    return sum(6.0 * tokens * k * n for (k, n, _, _) in spec['layers'])


def run_reference(args, spec, world_size, rank):
    """CPU arm: torch.nn.Linear + activation on all host cores, bounded sample of the workload."""
    if rank != 0:
        return
    from oracle.cpu_baseline import time_torch_cpu_linear
    sample_rows = 512
    seconds, threads = 0.0, 1
    for (k, n, act, bias) in spec['layers']:
        r = time_torch_cpu_linear(sample_rows, k, n, act, bias, None, args.steps, args.warmup)
        seconds += r['seconds_per_step']
        threads = r['threads']
    tflops = flops_per_step(spec, sample_rows) / seconds / 1e12
    sample = (f'{sample_rows} of the batch rows per step, torch.nn.Linear + activation fwd+bwd in fp32 '
              f'on {threads} host threads')
    line = {
        'impl': 'reference', 'metric': 'linear_fwd_bwd_tflops', 'value': tflops, 'unit': 'TFLOP/s',
        'n_gpus': world_size, 'steps': args.steps, 'warmup': args.warmup,
        'ms_per_step': seconds * 1e3, 'higher_is_better': True, 'scaling': spec['scaling'],
        'vs_baseline': None, 'dtype': 'f32', 'data': 'synthetic',
        'config': {'workload': args.workload, 'sample': sample},
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
    bo = torch.randn(n0, device=device).to(op_dtype)
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
            k0, 1, n0, 1, n0, n0, dt_id, dt_id, dt_id, act_id(name), param or 0.0, gws.data_ptr(), gws_bytes,
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


def kernel_only(args, spec, tokens, device, lib):
    """A few launches of one kernel and nothing else: the target of ncu captures."""
    launch, work, unit = kernel_launcher(spec, tokens, device, lib, args.kernel_only)
    for _ in range(max(args.warmup, 1)):
        launch()
    torch.cuda.synchronize()
    r0, r1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    r0.record()
    for _ in range(args.steps):
        launch()
    r1.record()
    torch.cuda.synchronize()
    ms = r0.elapsed_time(r1) / args.steps
    rate = {'tflops': work / (ms * 1e-3) / 1e12} if unit == 'flops' else {'gbs': work / (ms * 1e-3) / 1e9}
    print(json.dumps({'kernel_only': args.kernel_only, 'tokens': tokens, 'kernel_ms': ms, **rate}), flush=True)


def skinny_forward(args, device, lib):
    """
    BASELINE.json config 4: y = x @ W for fp16 x [M, 8192], W [8192, 28672], no bias, no activation, under
    torch.no_grad(), through the module.  HBM-bound: the score is algorithmic bytes
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
            for _ in range(max(args.warmup, 3)):
                layer(x)
            torch.cuda.synchronize()
            t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            t0.record()
            for _ in range(args.steps):
                layer(x)
            t1.record()
            torch.cuda.synchronize()
        ms = t0.elapsed_time(t1) / args.steps
        nbytes = 2.0 * (K * N + m * K + m * N)
        path = {_lib.PATH_STREAMK: 'memset + swap-AB stream-K tcgen05 + finish',
                _lib.PATH_TCGEN05: 'one wave of whole 128 x 256 tcgen05 tiles'}.get(lib.ab200_last_path(), 'other')
        rows.append({'M': m, 'us': ms * 1e3, 'gbs': nbytes / (ms * 1e-3) / 1e9, 'path': path,
                     'frac_of_measured_hbm': nbytes / (ms * 1e-3) / 1e9 / peaks['hbm_gbs'],
                     'frac_of_nominal_8000': nbytes / (ms * 1e-3) / 1e9 / 8000.0})
    attorch_b200.check_status()
    best = max(r['gbs'] for r in rows)
    print(json.dumps({'metric': 'skinny_forward_weight_read_gbs', 'value': best, 'unit': 'GB/s', 'n_gpus': 1,
                      'steps': args.steps, 'warmup': args.warmup, 'higher_is_better': True, 'dtype': 'f16',
                      'data': 'synthetic', 'config': {'workload': 'c4', 'K': K, 'N': N, 'rows': rows,
                                                      'call': 'attorch_b200.Linear under torch.no_grad()'},
                      'roofline': {'bound': 'hbm', 'achieved': best, 'peak': peaks['hbm_gbs'], 'unit': 'GB/s',
                                   'frac': best / peaks['hbm_gbs'], 'traffic': None,
                                   'peak_source': peak_source}}), flush=True)


def activation_layer(args, device):
    """
    The standalone activation layer with fused dropout (the row after the linear layer in the scope
    table): GELU with drop_p = 0.1 on a bf16 [32768, 4096] tensor (268 MB, larger than L2), forward and
    input gradient, timed through the C ABI (the kernels alone) and through attorch_b200.GELU (with
    the host work of the module around them).  HBM-bound: algorithmic bytes are 2 n e forward (read x,
    write y) and 3 n e backward (read dy and x, write dx).
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
        for _ in range(max(args.warmup, 3)):
            fn()
        torch.cuda.synchronize()
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0.record()
        for _ in range(args.steps):
            fn()
        t1.record()
        torch.cuda.synchronize()
        ms = t0.elapsed_time(t1) / args.steps
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
        for _ in range(max(args.warmup, 3)):
            fn()
        torch.cuda.synchronize()
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0.record()
        for _ in range(args.steps):
            fn()
        t1.record()
        torch.cuda.synchronize()
        ms = t0.elapsed_time(t1) / args.steps
        results[name] = {'us': round(ms * 1e3, 2), 'gbs': round(nbytes / (ms * 1e-3) / 1e9, 1)}
    best = results[args.only or 'kernel_forward']['gbs']
    print(json.dumps({'metric': 'activation_layer_gbs', 'value': best, 'unit': 'GB/s', 'n_gpus': 1,
                      'steps': args.steps, 'warmup': args.warmup, 'higher_is_better': True, 'dtype': 'bf16',
                      'data': 'synthetic',
                      'config': {'workload': 'act', 'layer': 'GELU(drop_p=0.1)', 'shape': [n_rows, n_cols],
                                 'l2': 'inputs larger than L2', **results},
                      'roofline': {'bound': 'hbm', 'achieved': best, 'peak': peaks['hbm_gbs'], 'unit': 'GB/s',
                                   'frac': best / peaks['hbm_gbs'], 'traffic': None, 'peak_source': peak_source}}),
          flush=True)


def main():
    parser = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawTextHelpFormatter)
    parser.add_argument('--gpus', type=int, default=1)
    parser.add_argument('--steps', type=int, default=200)
    parser.add_argument('--warmup', type=int, default=10)
    parser.add_argument('--workload', choices=sorted(WORKLOADS) + ['c4', 'act'], default='c2')
    parser.add_argument('--only', default=None,
                        help='workload act: time just this entry (e.g. kernel_forward, glu_backward)')
    parser.add_argument('--impl', choices=['b200', 'reference'], default='b200')
    parser.add_argument('--no-cpu-baseline', action='store_true')
    parser.add_argument('--no-graph', action='store_true',
                        help='launch every step eagerly instead of replaying one captured CUDA graph')
    parser.add_argument('--kernel-only', choices=['fwd', 'dx', 'dw', 'act_bwd'], default=None,
                        help='launch only this kernel of the first layer (for ncu captures)')
    parser.add_argument('--tokens', type=int, default=None,
                        help='override the tokens per GPU (profiling of reduced cases)')
    args = parser.parse_args()
    args.warmup = max(args.warmup, 3)
    if args.workload in ('c4', 'act'):
        if args.impl == 'reference':
            print(json.dumps({'impl': 'reference', 'unavailable': f'{args.workload} has no CPU arm; use c2'}))
            return
        from attorch_b200 import _lib
        torch.cuda.set_device(0)
        if args.workload == 'c4':
            skinny_forward(args, torch.device('cuda', 0), _lib.load())
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
    from attorch_b200.dp import GradientBuckets

    if not torch.cuda.is_available():
        raise SystemExit('bench.py needs a CUDA device: the layer has no CPU fallback')
    lib = _lib.load()
    torch.cuda.set_device(local_rank)
    device = torch.device('cuda', local_rank)
    if world_size > 1:
        os.environ.setdefault('MASTER_ADDR', '127.0.0.1')
        dist.init_process_group('nccl', device_id=device)

    tokens = args.tokens or spec['tokens_per_gpu'] or spec['global_tokens'] // world_size
    total_tokens = tokens * world_size
    torch.manual_seed(0)
    layers = [attorch_b200.Linear(k, n, bias=bias, act_func=act, device=device,
                                  dtype=spec['param_dtype'])
              for (k, n, act, bias) in spec['layers']]
    # One GPU: a step is one captured CUDA graph.  Several GPUs: NCCL cannot be captured here (see
    # below), so either the step is launched eagerly with the gradient exchange issued per block of dW
    # from inside backward, overlapping the rest of it (--no-graph; the default where a rank has at
    # least 4 host threads to itself), or the local computation is replayed from a graph and followed by
    # one all-reduce of the bucket.  Measured at 2 GPUs: eager overlapped 0.839-0.894 ms, graph + one
    # all-reduce 0.886-0.887 ms, eager without overlap 0.877 ms; at 8 GPUs eager overlapped 0.959 ms
    # (1.001 ms on a box with 2 host threads per rank, where enqueueing takes 0.91 ms per step).
    # AB200_DEFER_DX=1 selects a third schedule: two graphs per step with the all-reduce started between
    # them, so that it overlaps the first layer's dX (which runs on 16 fewer SMs).  It measured slower
    # at 2 GPUs (0.914-0.924 ms): the exchange and the GEMM slow each other down more than the overlap
    # saves.
    if world_size > 1 and (os.cpu_count() or 1) // world_size >= 4 and not os.environ.get('AB200_FORCE_GRAPH') \
            and os.environ.get('AB200_DEFER_DX', '0') != '1':
        args.no_graph = True
    defer = world_size > 1 and not args.no_graph and os.environ.get('AB200_DEFER_DX', '0') == '1'
    overlap = args.no_graph and os.environ.get('AB200_DP_OVERLAP', '1') != '0'
    buckets = GradientBuckets(layers, comm_sms=int(os.environ.get('AB200_COMM_SMS', '16')),
                              overlap=overlap, defer_first_input_grad=defer,
                              dw_chunks=int(os.environ.get('AB200_DW_CHUNKS', '2')))
    k_in, n_out = spec['layers'][0][0], spec['layers'][-1][1]
    gen = torch.Generator(device=device).manual_seed(1 + rank)
    x_dev = torch.randn(tokens, k_in, device=device, generator=gen).to(spec['input_dtype'])
    x_dev.requires_grad_(True)
    out_dtype = spec['autocast'] or spec['param_dtype']
    dy = (torch.randn(tokens, n_out, device=device, generator=gen) * 0.01).to(out_dtype)

    def compute(x):
        buckets.zero_grad()
        x.grad = None
        with torch.autocast('cuda', dtype=spec['autocast'] or torch.bfloat16,
                            enabled=spec['autocast'] is not None):
            h = x
            for layer in layers:
                h = layer(h)
        h.backward(dy)

    def deferred_products():
        # The GEMMs held back run beside the exchange: leave NCCL some SMs.
        lib.ab200_set_gemm_cta_limit(buckets.exchange_cta_limit())
        try:
            buckets.run_deferred()
        finally:
            lib.ab200_set_gemm_cta_limit(0)

    def step(x):
        compute(x)
        if defer:
            buckets.start_exchange()
            deferred_products()
        buckets.finish()

    def barrier():
        if world_size > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(ms):
        if world_size == 1:
            return ms
        t = torch.tensor([ms], dtype=torch.float64, device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    if args.kernel_only:
        kernel_only(args, spec, tokens, device, lib)
        return

    # ---------------------------------------------------------------- device-resident timing
    for _ in range(args.warmup):
        step(x_dev)
    barrier()
    attorch_b200.check_status()

    # One step (forward, backward, gradient exchange) captured once as a CUDA graph and replayed:
    # the same kernels on the same buffers, without the host-side gaps between launches.
    run_step, graphed = (lambda: step(x_dev)), False
    if not args.no_graph:
        # Only the local computation is captured: capturing the NCCL all-reduce as well (on the
        # harness's side stream) did not return within 600 s on this pool.
        try:
            side = torch.cuda.Stream(device)
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                for _ in range(3):
                    step(x_dev)
            torch.cuda.current_stream().wait_stream(side)
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                compute(x_dev)
            tail_graph = None
            if defer:
                tail_graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(tail_graph, pool=graph.pool()):
                    deferred_products()

            def run_step():
                graph.replay()
                if tail_graph is not None:
                    buckets.start_exchange()
                    tail_graph.replay()
                buckets.finish()
            run_step()
            torch.cuda.synchronize()
            attorch_b200.check_status()
            graphed = True
        except Exception as error:  # capture unsupported here: time the eager loop instead
            print(f'CUDA graph capture failed, timing eager launches: {error}', file=sys.stderr)
            torch.cuda.synchronize()
    for _ in range(3):
        run_step()
    barrier()
    launches_before = lib.ab200_launch_count()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(local_rank if rank == 0 else -1) as clocks:
        barrier()
        start.record()
        host_t0 = time.perf_counter()
        for _ in range(args.steps):
            run_step()
        host_ms_per_step = (time.perf_counter() - host_t0) * 1e3 / args.steps
        stop.record()
        barrier()
    launches = lib.ab200_launch_count() - launches_before
    if graphed:
        # Replays do not pass through the library's host code: count one eager step instead.
        before = lib.ab200_launch_count()
        step(x_dev)
        torch.cuda.synchronize()
        launches = (lib.ab200_launch_count() - before) * args.steps
    ms_total = max_over_ranks(start.elapsed_time(stop))
    attorch_b200.check_status()
    ms_per_step = ms_total / args.steps
    step_flops = flops_per_step(spec, tokens)
    value = step_flops * world_size / (ms_per_step * 1e-3) / 1e12

    # ---------------------------------------------------------------- end to end with host buffers
    host_x = [torch.randn(tokens, k_in).to(spec['input_dtype']).pin_memory() for _ in range(2)]
    dev_x = [torch.empty_like(x_dev).requires_grad_(True) for _ in range(2)]
    # The step's result that is read back: the last layer's bias gradient, or, for a layer without
    # bias, the first row of its weight gradient.
    def result_tensor():
        last = layers[-1]
        return last.bias.grad if last.bias is not None else last.weight.grad[0]
    bias_grad_host = torch.empty(n_out, dtype=spec['param_dtype']).pin_memory()
    copy_stream = torch.cuda.Stream(device)
    copied = [torch.cuda.Event() for _ in range(2)]
    consumed = [torch.cuda.Event() for _ in range(2)]

    def e2e_loop(n_steps):
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
            step(dev_x[cur])
            consumed[cur].record(compute)
            bias_grad_host.copy_(result_tensor(), non_blocking=True)
        compute.synchronize()

    e2e_loop(3)
    barrier()
    e2e_steps = max(10, min(args.steps, 40))
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0.record()
    e2e_loop(e2e_steps)
    t1.record()
    barrier()
    e2e_ms = max_over_ranks(t0.elapsed_time(t1)) / e2e_steps
    e2e_value = step_flops * world_size / (e2e_ms * 1e-3) / 1e12
    attorch_b200.check_status()

    # ---------------------------------------------------------------- roofline of the dominant kernel
    # The tcgen05 GEMM, launched through the C ABI exactly as the layer launches it (forward of the
    # first layer: X[M, K] * W[K, N] with bias, gelu and the pre-activation store), event-timed on
    # the launching stream.
    peaks, peak_source = measured_peaks()
    k0, n0 = spec['layers'][0][0], spec['layers'][0][1]
    launch_fwd, _, _ = kernel_launcher(spec, tokens, device, lib, 'fwd')

    for _ in range(5):
        launch_fwd()
    torch.cuda.synchronize()
    reps = 30
    r0, r1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    r0.record()
    for _ in range(reps):
        launch_fwd()
    r1.record()
    torch.cuda.synchronize()
    kernel_ms = r0.elapsed_time(r1) / reps
    achieved = 2.0 * tokens * k0 * n0 / (kernel_ms * 1e-3) / 1e12
    roofline = {'bound': 'tensor', 'achieved': achieved, 'peak': peaks['bf16_tflops'], 'unit': 'TFLOP/s',
                'frac': achieved / peaks['bf16_tflops'],
                'traffic': NCU_DRAM_BYTES_PER_LAUNCH if (args.workload == 'c2' and tokens == 8192) else None,
                'kernel': 'gemm_tcgen05_kernel (forward: bias + gelu + saved-derivative epilogue)',
                'kernel_ms': kernel_ms, 'peak_source': f'{peak_source} (cuBLAS bf16 burst)',
                'frac_of_nominal_2250': achieved / 2250.0}

    if rank != 0:
        if world_size > 1:
            dist.destroy_process_group()
        return

    line = {
        'metric': 'linear_fwd_bwd_tflops', 'value': value, 'unit': 'TFLOP/s', 'n_gpus': world_size,
        'steps': args.steps, 'warmup': args.warmup, 'ms_per_step': ms_per_step,
        'host_enqueue_ms_per_step': host_ms_per_step,
        'higher_is_better': True, 'scaling': spec['scaling'], 'vs_baseline': None,
        'dtype': 'bf16', 'data': 'synthetic',
        'config': {'workload': args.workload,
                   'layers': [f'{k}->{n} act={act} bias={bias}' for (k, n, act, bias) in spec['layers']],
                   'tokens_per_gpu': tokens, 'global_tokens': total_tokens,
                   'params': str(spec['param_dtype']).replace('torch.', ''),
                   'input': str(spec['input_dtype']).replace('torch.', ''),
                   'autocast': str(spec['autocast']).replace('torch.', ''),
                   'parallelism': f'dp{world_size}',
                   'collective': ('none' if world_size == 1 else
                                  'NCCL all-reduce of dW/db, ' + (
                                      'issued per dW block inside backward, overlapped' if overlap else
                                      'one call between the two captured graphs of a step, overlapping the first '
                                      "layer's dX" if defer and graphed else 'one call after the step')),
                   'cuda_graph': graphed,
                   'l2': 'per-step working set (operands, activations, gradients) exceeds the 126 MB L2; no flush',
                   'tflops_per_gpu': value / world_size,
                   'frac_of_nominal_2250_per_gpu': value / world_size / 2250.0},
        'clocks': clocks.summary(),
        'e2e': {'value': e2e_value, 'unit': 'TFLOP/s', 'ms_per_step': e2e_ms,
                'h2d_bytes_per_step': host_x[0].numel() * host_x[0].element_size(),
                'd2h_bytes_per_step': bias_grad_host.numel() * bias_grad_host.element_size()},
        'gpu_launches': int(launches),
        'roofline': roofline,
    }
    if world_size == 1 and not args.no_cpu_baseline:
        from oracle.cpu_baseline import time_torch_cpu_linear
        sample_rows, seconds, threads = 512, 0.0, 1
        for (k, n, act, bias) in spec['layers']:
            r = time_torch_cpu_linear(sample_rows, k, n, act, bias, None, steps=10, warmup=2)
            seconds += r['seconds_per_step']
            threads = r['threads']
        line['cpu_baseline'] = {
            'value': flops_per_step(spec, sample_rows) / seconds / 1e12, 'unit': 'TFLOP/s', 'cores': threads,
            'kind': 'port',
            'sample': f'{sample_rows} of the batch rows per step, 10 steps, torch.nn.Linear + activation '
                      f'fwd+bwd in fp32 on {threads} host threads'}
    print(json.dumps(line), flush=True)
    if world_size > 1:
        dist.destroy_process_group()


if __name__ == '__main__':
    main()
