"""Benchmark of the block-sparse attention hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload (config.workload): sparse self-attention forward + backward, FP16,
Z=8, H=16, L=8192, head_dim 64, block 64, "fixed" layout (local windows of 4
blocks, last block of every window global, unidirectional) -- the configuration
the headline metric is quoted on.  Inputs are seeded synthetic N(0,1) tensors of
that shape (the reference measures on no dataset): batch entry z is drawn from
torch.Generator(seed = z), so every rank count sees the same problem.

One "step" is one forward + backward through the public wrapper
(SparseSelfAttention), captured once in a CUDA graph by its graphed() method and
replayed (the eager, call-by-call time is reported beside it).  `value` counts only the FLOPs of nonzero blocks
(6 products of 2*Z*nnz*block^2*D; softmax and recomputation are not counted)
with inputs resident in HBM; `e2e` is the same step on operands in pinned host
memory through the library's host entry (HostAttention): every step copies its
inputs in and its four results out inside the timed region, streamed by batch
slices so that transfers and kernels overlap.

With N > 1 the ONE problem above is split over the ranks by (batch, head)
shards (torch_blocksparse_b200.shard.plan: Z first, then H), no collective on
the timed path: strong scaling, `value` = FLOPs of the whole problem / the
slowest rank's time.  Off the clock the outputs and gradients of all ranks are
all-gathered over NCCL into full tensors and sampled (batch, head) slices are
compared with the CPU oracle.  Two secondary measurements at N > 1: `head_split`
(a problem of N/2 batch entries, so that every batch entry is split over the
heads of two ranks: layout slices, re-based tables) and `weak` (every rank runs
a full Z=8 problem of its own).  At N = 1 the line also carries the other
configurations: C4 bidirectional, C5 (BigBird, BF16, Z=32), C3 softmax, C1 / C2
and the large-block MatMul cases.

`--impl reference` times the reference's dense-masked definition of the same
op on the host cores (the CPU restatement under oracle/; nothing of the
product is imported), on a bounded sample of (batch, head) slices.
"""
import argparse
import json
import math
import os
import statistics
import subprocess
import sys
import tempfile
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

import workloads  # noqa: E402

METRIC = 'sparse_attn_fwd_bwd_tflops_nnz_blocks_L8192'
UNIT = 'TFLOP/s'
FALLBACK_PEAKS = {'hbm_gbs': 6650.0, 'bf16_tflops': 1590.0, 'bf16_tflops_sustained': 1400.0}
Z_TOTAL, HEADS, SEQ, HEAD_DIM, BLOCK = 8, 16, 8192, 64, 64

# dram__bytes_read.sum + dram__bytes_write.sum per launch from the ncu captures summarised
# under profiles/.  The attention figures were captured at Z=2 and are scaled to the launch's
# batch: every (batch, head) pair is independent, so traffic grows in proportion.
NCU_TRAFFIC_BYTES_PER_Z = {'attn_bwd_dkdv': 225.8e6 / 2, 'attn_fwd': 115.7e6 / 2, 'attn_bwd_dq': 154.3e6 / 2}
NCU_TRAFFIC_BYTES = {'softmax_fwd': 638.5e6, 'softmax_bwd': 924.3e6}


def peaks():
    path = os.path.join(ROOT, 'MEASURED_PEAKS.json')
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        p['source'] = 'measured'
        return p
    p = dict(FALLBACK_PEAKS)
    p['source'] = 'fallback'
    return p


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while active."""
    FIELDS = ('index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,'
              'clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,'
              'clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap')

    def __init__(self, index):
        self.index = index
        self.proc = None
        self.path = None

    def start(self):
        try:
            fd, self.path = tempfile.mkstemp(suffix='.csv')
            os.close(fd)
            self.proc = subprocess.Popen(['nvidia-smi', '-i', str(self.index), '--query-gpu=' + self.FIELDS,
                                          '--format=csv,noheader,nounits', '-lms', '100'],
                                         stdout=open(self.path, 'w'), stderr=subprocess.DEVNULL)
            time.sleep(0.3)
        except Exception:
            self.proc = None

    def stop(self):
        out = {'sm_mhz': None, 'sm_max_mhz': None, 'reasons': [], 'samples': 0}
        if self.proc is None:
            return out
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        try:
            for line in open(self.path):
                f = [x.strip() for x in line.split(',')]
                if len(f) < 9:
                    continue
                try:
                    sm.append(float(f[1]))
                    mx.append(float(f[2]))
                except ValueError:
                    continue
                for name, v in zip(('hw_slowdown', 'hw_thermal_slowdown', 'sw_thermal_slowdown', 'sw_power_cap'), f[5:9]):
                    if v.lower().startswith('active'):
                        reasons.add(name)
            os.unlink(self.path)
        except Exception:
            pass
        if sm:
            out.update(sm_mhz=statistics.median(sm), sm_max_mhz=max(mx), reasons=sorted(reasons), samples=len(sm))
        return out


def dist_env():
    rank = int(os.environ.get('RANK', 0))
    world = int(os.environ.get('WORLD_SIZE', 1))
    local = int(os.environ.get('LOCAL_RANK', 0))
    return rank, world, local


def problem_entries(attention, zs, h0=0, h1=HEADS):
    """Batch entries `zs` of the benchmark problem (entry z is drawn from seed z), heads [h0, h1):
    dict with q, k, v, do [len(zs), h1-h0, L, D] and the layout slice."""
    parts = [workloads.config4(attention, Z=1, seed=z) for z in zs]
    c = {n: torch.cat([p[n][:, h0:h1] for p in parts]).contiguous() for n in ('q', 'k', 'v', 'do')}
    c.update(layout=parts[0]['layout'][h0:h1].contiguous(), full_layout=parts[0]['layout'], block=parts[0]['block'],
             scale=parts[0]['scale'])
    return c


def cpu_attention_sample(attention, n_slices, Z=Z_TOTAL):
    """Times the dense-masked CPU definition on `n_slices` (batch, head) slices of the
    workload.  Returns (seconds for the sample, counted FLOPs of the sample)."""
    from oracle import dense_masked as dm
    slices = [(i % Z, (i * 7) % HEADS) for i in range(n_slices)]
    data = {}
    for z in sorted({z for z, _ in slices}):
        data[z] = workloads.config4(attention, Z=1, seed=z)
    flops = 0
    t0 = time.perf_counter()
    for z, h in slices:
        c = data[z]
        flops += workloads.attention_flops(c['layout'][h:h + 1], c['block'], 1, c['q'].size(-1))
        dm.attention_reference(c['q'][:, h:h + 1], c['k'][:, h:h + 1], c['v'][:, h:h + 1],
                               c['layout'][h:h + 1], c['block'], c['scale'], do=c['do'][:, h:h + 1])
    return time.perf_counter() - t0, flops


def config_dict(args, world, n_sets=1):
    return {'workload': 'config4: sparse self-attention fwd+bwd FP16, Z=%d, H=16, L=8192, head_dim=64, block=64, '
                        'fixed layout (windows of 4 blocks, last block global), %s' % (Z_TOTAL, args.attention),
            'global_batch': Z_TOTAL, 'seq_len': SEQ, 'heads': HEADS, 'head_dim': HEAD_DIM, 'block': BLOCK,
            'parallelism': 'one problem split into (batch, head) shards over %d GPU(s), no collective on the timed path'
                           % world,
            'l2': ('inputs (4 x 134 MB) exceed the 126 MB L2; no explicit flush' if n_sets == 1 else
                   'the shard is smaller than L2: steps rotate over %d copies of the inputs (> 400 MB in all), '
                   'no explicit flush' % n_sets)}


def run_reference(args):
    rank, world, _ = dist_env()
    if rank != 0:
        return
    workloads.LAYOUT_SOURCE = 'oracle'          # nothing of the product is imported on this arm
    torch.set_num_threads(os.cpu_count() or 1)
    n_slices = args.ref_slices
    for _ in range(min(args.warmup, 1)):
        cpu_attention_sample(args.attention, n_slices)
    flops, dt = 0, 0.0
    for _ in range(args.steps):                 # (drawing the inputs is not part of a step's time)
        t, f = cpu_attention_sample(args.attention, n_slices)
        flops += f
        dt += t
    value = flops / dt / 1e12
    sample = ('%d of the %d (batch, head) slices per step, dense-masked FP32 torch on FP16-rounded inputs'
              % (n_slices, Z_TOTAL * HEADS))
    line = {
        'impl': 'reference', 'metric': METRIC, 'value': value, 'unit': UNIT, 'n_gpus': args.gpus,
        'steps': args.steps, 'warmup': args.warmup, 'ms_per_step': dt / args.steps * 1e3,
        'higher_is_better': True, 'scaling': 'strong', 'vs_baseline': None, 'dtype': 'f32', 'data': 'synthetic',
        'config': config_dict(args, world),
        'cpu_baseline': {'value': value, 'unit': UNIT, 'cores': torch.get_num_threads(), 'kind': 'port', 'sample': sample},
        'e2e': {'value': value, 'unit': UNIT, 'h2d_bytes_per_step': 0, 'd2h_bytes_per_step': 0},
        'gpu_launches': 0,
    }
    print(json.dumps(line))


# ---------------------------------------------------------------------------------------------
# our arm
# ---------------------------------------------------------------------------------------------
class Timing:
    """Shared timing helpers of one rank: barrier + synchronize on both sides, CUDA events on the
    current stream, max over ranks."""

    def __init__(self, dev, world):
        self.dev, self.world = dev, world

    def barrier(self):
        if self.world > 1:
            import torch.distributed as dist
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(self, seconds):
        el = torch.tensor([seconds], device=self.dev, dtype=torch.float64)
        if self.world > 1:
            import torch.distributed as dist
            dist.all_reduce(el, op=dist.ReduceOp.MAX)
        return float(el)

    def run(self, step, steps, warmup=3, profile=False):
        """`steps` calls of step(i) between two events.  Returns (seconds as the max over ranks,
        per-kernel event triples when profile)."""
        from torch_blocksparse_b200 import fused
        fused.PROFILE = [] if profile else None
        for i in range(warmup):
            step(i)
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        fused.PROFILE = [] if profile else None
        self.barrier()
        t0.record()
        for i in range(steps):
            step(i)
        t1.record()
        self.barrier()
        prof, fused.PROFILE = fused.PROFILE, None
        return self.max_over_ranks(t0.elapsed_time(t1) * 1e-3), prof


def make_steps(mod, c, dev, n_sets):
    """Device copies of the shard's inputs (n_sets of them, rotated step by step so that a small
    shard does not live in L2) and the step function: forward + backward through the module."""
    sets = []
    for _ in range(n_sets):
        q, k, v = (c[n].to(dev).requires_grad_() for n in ('q', 'k', 'v'))
        sets.append((q, k, v, c['do'].to(dev)))
    state = {}

    def step(i):
        q, k, v, do = sets[i % n_sets]
        q.grad = k.grad = v.grad = None
        o = mod(q, k, v)
        o.backward(do)
        state['last'] = (o.detach(), q.grad, k.grad, v.grad)
        return o

    # the same step captured once per input set in a CUDA graph (module.graphed) and replayed
    graphs = [mod.graphed(q.detach(), k.detach(), v.detach(), do) for q, k, v, do in sets]

    def graphed_step(i):
        g = graphs[i % n_sets]
        g.replay()
        state['last'] = (g.o, g.dq, g.dk, g.dv)

    state['graphed'] = graphed_step
    return step, state


def attention_section(name, c, dev, steps, pk, T, dtype_name, **extra):
    """One-GPU timing of a whole configuration (extra keys of the N = 1 line); `extra`: rpe / masks
    handed to the attention call."""
    from torch_blocksparse_b200 import SparseSelfAttention
    layout, block = c['layout'], c['block']
    Z, _, L, D = c['q'].shape
    mod = SparseSelfAttention(layout=layout, block=block, fused=True)
    q, k, v = (c[n].to(dev).requires_grad_() for n in ('q', 'k', 'v'))
    do = c['do'].to(dev)

    def step(i):
        q.grad = k.grad = v.grad = None
        mod(q, k, v, **extra).backward(do)

    _, prof = T.run(step, max(2, steps // 2), warmup=3, profile=True)      # per-kernel durations
    t, _ = T.run(step, steps, warmup=2, profile=False)                     # the step as a user issues it
    flops = workloads.attention_flops(layout, block, Z, D)
    kern = {}
    for n, a, b in prof:
        kern.setdefault(n, []).append(a.elapsed_time(b))
    kern_ms = {n: sum(x) / len(x) for n, x in kern.items()}
    top = max(kern_ms, key=kern_ms.get)
    per_product = 2 * Z * int(layout.sum()) * block * block * D
    counted = {'attn_fwd': 2, 'attn_bwd_dkdv': 2, 'attn_bwd_dq': 1, 'attn_bwd_delta': 0, 'attn_bwd_fused': 3}
    ach = counted.get(top, 0) * per_product / (kern_ms[top] * 1e-3) / 1e12
    return {'workload': name, 'tflops': flops / t * steps / 1e12, 'ms_per_step': t / steps * 1e3, 'dtype': dtype_name,
            'kernel_ms': kern_ms, 'frac_of_nominal_peak': flops / t * steps / 1e12 / 2250.0,
            'roofline': {'bound': 'tensor', 'kernel': top, 'achieved': ach, 'peak': pk['bf16_tflops'], 'unit': UNIT,
                         'frac': ach / pk['bf16_tflops'], 'traffic': None,
                         'peak_source': pk['source'] + ' (bf16 dense, burst)'},
            'gpu_launches': steps * 4}


def matmul_bench(dev, pk, iters=10, z=8, section='all'):
    """Block-sparse MatMul: configuration 1 (sdd FP32 block 16), configuration 2 (dsd / dds, FP16,
    block 32, Z=8, H=8, 2048^3, layout Bernoulli(0.25)) forward and forward + backward, and blocks
    64 / 128 on a compute-bound shape; TFLOP/s on nonzero-block FLOPs."""
    from torch_blocksparse_b200 import MatMul
    out = {'workload': 'config2: dsd / dds FP16, block 32, Z=%d, H=8, M=N=K=2048, Bernoulli(0.25) layout' % z, 'cases': []}
    peak_tf = pk['bf16_tflops']

    def timed(fn):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(iters):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / iters * 1e-3

    if section == 'large':
        return large_blocks_bench(dev, pk, timed, out)
    c1 = workloads.config1()
    op = MatMul(c1['layout'], 16, 'sdd', trans_a=True, trans_b=False)
    a, b = c1['a'].to(dev), c1['b'].to(dev)
    t = timed(lambda: op(a, b))
    nnz = int(c1['layout'].sum())
    fl = 2 * 4 * nnz * 16 * 16 * 384
    by = 4 * (a.numel() + b.numel() + 4 * nnz * 256)
    out['config1'] = {'workload': 'config1: sdd FP32 block 16, trans_a, A [4,2,384,256], B [4,2,384,512], Bernoulli(0.5) layout',
                      'fwd_ms': t * 1e3, 'fwd_tflops': fl / t / 1e12, 'fwd_gbs': by / t / 1e9,
                      'note': '0.40 GFLOP and 5.3 MB: one launch of a few microseconds, bound by launch latency'}

    for mode in ('dsd', 'dds'):
        for ta in (False, True):
            for tb in (False, True):
                c = workloads.config2(mode, ta, tb)
                op = MatMul(c['layout'], c['block'], mode, trans_a=ta, trans_b=tb)
                a = c['a'][:z].to(dev).requires_grad_()
                b = c['b'][:z].to(dev).requires_grad_()
                dc = c['dc'][:z].to(dev)
                flops = 2 * z * int(c['layout'].sum()) * c['block'] ** 2 * 2048

                def fwd_bwd():
                    a.grad = b.grad = None
                    op(a, b).backward(dc)

                tf, tfb = timed(lambda: op(a, b)), timed(fwd_bwd)
                out['cases'].append({'mode': mode, 'trans_a': ta, 'trans_b': tb, 'fwd_ms': tf * 1e3,
                                     'fwd_tflops': flops / tf / 1e12, 'fwd_bwd_ms': tfb * 1e3,
                                     'fwd_bwd_tflops': 3 * flops / tfb / 1e12,
                                     'fwd_frac_of_measured_peak': flops / tf / 1e12 / peak_tf})
                del a, b, dc, c
                torch.cuda.empty_cache()
    best = max(out['cases'], key=lambda e: e['fwd_tflops'])
    worst = min(out['cases'], key=lambda e: e['fwd_tflops'])
    out['roofline'] = {'bound': 'tensor', 'kernel': 'dsd_tc_kernel (block 32)', 'achieved': worst['fwd_tflops'],
                       'achieved_best': best['fwd_tflops'], 'peak': peak_tf, 'unit': UNIT,
                       'frac': worst['fwd_tflops'] / peak_tf, 'traffic': None,
                       'peak_source': pk['source'] + ' (bf16 dense, burst)'}
    if section == 'config2':
        return out
    return large_blocks_bench(dev, pk, timed, out)


def large_blocks_bench(dev, pk, timed, out):
    from torch_blocksparse_b200 import MatMul
    peak_tf = pk['bf16_tflops']
    # blocks 64 and 128 (the tcgen05 kernels) on a compute-bound shape: Z=2, H=8, M=N=K=4096,
    # layout Bernoulli(0.25), forward only, every mode, plain and one transposed variant
    out['large_blocks'] = {'workload': 'sdd / dsd / dds FP16, block 64 and 128, Z=2, H=8, M=N=K=4096, Bernoulli(0.25) layout, forward',
                           'cases': []}
    S, zz, hh = 4096, 2, 8
    g = torch.Generator().manual_seed(0)
    for block in (64, 128):
        nb = S // block
        layout = (torch.rand((hh, nb, nb), generator=g) < 0.25).long()
        nnz = int(layout.sum())
        d1 = (torch.randn((zz, hh, S, S), generator=g) * S ** -0.5).half().to(dev)
        d2 = (torch.randn((zz, hh, S, S), generator=g) * S ** -0.5).half().to(dev)
        sp = (torch.randn((zz, nnz, block, block), generator=g) * S ** -0.5).half().to(dev)
        flops = 2 * zz * nnz * block * block * S
        for mode, a, b in (('sdd', d1, d2), ('dsd', sp, d1), ('dds', d1, sp)):
            for ta, tb in ((False, False), (True, False), (False, True)):
                op = MatMul(layout, block, mode, trans_a=ta, trans_b=tb)
                t = timed(lambda: op(a, b))
                out['large_blocks']['cases'].append({'block': block, 'mode': mode, 'trans_a': ta, 'trans_b': tb, 'fwd_ms': t * 1e3,
                                                     'fwd_tflops': flops / t / 1e12,
                                                     'fwd_frac_of_measured_peak': flops / t / 1e12 / peak_tf})
        del d1, d2, sp
        torch.cuda.empty_cache()
    # the same shape on a banded layout of the same density (every block-row sees the 25 % of the
    # block-columns around its own): neighbouring rows share their columns, so a tile's union of
    # column lists holds little that is not in the layout
    from torch_blocksparse_b200 import layouts
    out['banded'] = {'workload': 'sdd / dsd / dds FP16, block 32, 64 and 128, Z=2, H=8, M=N=K=4096, band of a quarter of '
                                 'the block-columns around the diagonal, forward', 'cases': []}
    for block in (32, 64, 128):
        nb = S // block
        layout = layouts.window(hh, nb, nb // 8, nb // 8 - 1)
        nnz = int(layout.sum())
        d1 = (torch.randn((zz, hh, S, S), generator=g) * S ** -0.5).half().to(dev)
        d2 = (torch.randn((zz, hh, S, S), generator=g) * S ** -0.5).half().to(dev)
        sp = (torch.randn((zz, nnz, block, block), generator=g) * S ** -0.5).half().to(dev)
        flops = 2 * zz * nnz * block * block * S
        for mode, a, b in (('sdd', d1, d2), ('dsd', sp, d1), ('dds', d1, sp)):
            op = MatMul(layout, block, mode)
            t = timed(lambda: op(a, b))
            out['banded']['cases'].append({'block': block, 'mode': mode, 'fwd_ms': t * 1e3, 'fwd_tflops': flops / t / 1e12,
                                           'fwd_frac_of_measured_peak': flops / t / 1e12 / peak_tf})
        del d1, d2, sp
        torch.cuda.empty_cache()
    return out


def softmax_bench(dev, pk, iters=20):
    """Sparse softmax (configuration 3) forward / backward bandwidth: through the raw C ABI and
    through the public op (Softmax.__call__ and its autograd backward)."""
    from torch_blocksparse_b200 import Softmax
    c = workloads.config3()
    layout, block = c['layout'], c['block']
    op = Softmax(layout, block)
    x = c['x'].to(dev)
    dy = c['dy'].to(dev)
    rpe = c['rpe'].to(dev)[None].expand(x.size(0), -1, -1, -1)
    kpm, am = c['key_padding_mask'].to(dev), c['attn_mask'].to(dev)
    lut, maxlut = op.make_lut(x.device)
    from torch_blocksparse_b200 import _lib
    from torch_blocksparse_b200.matmul import _dtype_code, _stream
    H, Mb, _ = layout.shape
    L = _lib.lib()

    def fwd():
        _lib.check(L.bsp_softmax_fwd(x.data_ptr(), _dtype_code(x), x.size(0), x.stride(0), block, H, Mb,
                                     lut.data_ptr(), maxlut, c['scale'], rpe.data_ptr(), 0, rpe.stride(1), rpe.stride(2),
                                     kpm.data_ptr(), kpm.stride(0), 0, am.data_ptr(), am.stride(0), 1, _stream(x)))

    def bwd():
        _lib.check(L.bsp_softmax_bwd(x.data_ptr(), dy.data_ptr(), _dtype_code(x), x.size(0), x.stride(0), dy.stride(0),
                                     block, H, Mb, lut.data_ptr(), maxlut, c['scale'], _stream(x)))

    def op_fwd():
        with torch.no_grad():
            op(x, scale=c['scale'], rpe=rpe, key_padding_mask=kpm, attn_mask=am,
               key_padding_mask_mode='add', attn_mask_mode='mul')

    def timeit(fn):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0.record()
        for _ in range(iters):
            fn()
        t1.record()
        torch.cuda.synchronize()
        return t0.elapsed_time(t1) / iters * 1e-3

    nnz = int(layout.sum())
    nnz_head = nnz // H
    e = 2
    xb = x.numel() * e
    fwd_bytes = 2 * xb + nnz * block * block * e + nnz_head * block * block * e + kpm.numel() * e
    bwd_bytes = 3 * xb
    tf, tb, tof = timeit(fwd), timeit(bwd), timeit(op_fwd)
    return {
        'workload': 'config3: FP16, block 64, Z=8, H=16, 4096x4096, causal band of 4 + first column, scale, rpe, '
                    'key-padding mask (add), causal mask (mul)',
        'fwd_gbs': fwd_bytes / tf / 1e9, 'bwd_gbs': bwd_bytes / tb / 1e9,
        'fwd_ms': tf * 1e3, 'bwd_ms': tb * 1e3, 'fwd_bytes': fwd_bytes, 'bwd_bytes': bwd_bytes,
        'op_call_fwd_gbs': fwd_bytes / tof / 1e9, 'op_call_fwd_ms': tof * 1e3,
        'frac_of_8tbs': fwd_bytes / tf / 1e9 / 8000.0,
        'roofline': {'bound': 'hbm', 'achieved': fwd_bytes / tf / 1e9, 'peak': pk['hbm_gbs'], 'unit': 'GB/s',
                     'frac': fwd_bytes / tf / 1e9 / pk['hbm_gbs'], 'traffic': NCU_TRAFFIC_BYTES['softmax_fwd'],
                     'kernel': 'softmax_fwd', 'peak_source': pk['source']},
        'roofline_bwd': {'bound': 'hbm', 'achieved': bwd_bytes / tb / 1e9, 'peak': pk['hbm_gbs'], 'unit': 'GB/s',
                         'frac': bwd_bytes / tb / 1e9 / pk['hbm_gbs'], 'traffic': NCU_TRAFFIC_BYTES['softmax_bwd'],
                         'kernel': 'softmax_bwd_group', 'peak_source': pk['source']},
        'gpu_launches': 3 * (iters + 3),
    }


def table_build_times(dev):
    """One-off costs of the layout-derived data for the configuration-4 layout (milliseconds):
    the three reference-format tables and the kernels' metadata on the host, the metadata on the
    device, the attention tile lists.  The reference spends 0.2 - 0.35 s in its Python builders
    for this layout (measured on its own code, CPU only)."""
    from torch_blocksparse_b200 import layouts, tables
    layout = layouts.fixed(HEADS, SEQ // BLOCK, 4, 'unidirectional')

    def ms(fn, n=3):
        best = None
        for _ in range(n):
            tables.clear_cache()
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            fn()
            torch.cuda.synchronize()
            dt = (time.perf_counter() - t0) * 1e3
            best = dt if best is None else min(best, dt)
        return best

    lay_dev = layout.to(dev)
    out = {'layout': 'config4 unidirectional [16,128,128], 36 864 blocks',
           'reference_tables_host_ms': ms(lambda: (tables.make_sdd_lut(layout, BLOCK), tables.make_dxx_lut(layout, BLOCK, 16, False),
                                                   tables.make_dxx_lut(layout, BLOCK, 16, True), tables.make_softmax_lut(layout))),
           'metadata_host_build_and_upload_ms': ms(lambda: tables.build_meta(layout).on(dev)),
           'metadata_device_build_ms': ms(lambda: tables.build_meta_device(lay_dev)),
           'attention_tiles_host_build_and_upload_ms': ms(lambda: tables.build_attn_tiles(layout, BLOCK).on(dev)),
           'cached_lookup_ms': None}
    tables.build_meta(layout)
    t0 = time.perf_counter()
    tables.build_meta(layout)
    out['cached_lookup_ms'] = (time.perf_counter() - t0) * 1e3
    return out


def oracle_check(gathered, entries, slices):
    """Compares (batch, head) slices of the gathered o, dq, dk, dv with the CPU oracle on the
    problem's own inputs.  `entries`: {z: config dict of batch entry z}.  Returns the largest
    error in units of the tolerance (<= 1 passes) and the slices."""
    from oracle import dense_masked as dm
    worst = 0.0
    for z, h in slices:
        c = entries[z]
        want = dm.attention_reference(c['q'][:, h:h + 1], c['k'][:, h:h + 1], c['v'][:, h:h + 1], c['layout'][h:h + 1],
                                      c['block'], c['scale'], do=c['do'][:, h:h + 1])
        for g, w in zip(gathered, want):
            got = g[z:z + 1, h:h + 1].float().cpu()
            w = w.float()
            worst = max(worst, float(((got - w).abs() / (1e-2 + 1e-2 * w.abs())).max()))
    return worst


def run_sharded(args, T, dev, rank, world, Z, pk, profile, n_slices_checked=2, sampler=None):
    """Splits the problem of batch entries 0..Z-1 over the ranks, times `steps` steps of every
    rank's shard and (world > 1) gathers the results and checks them.  Returns a dict."""
    import torch.distributed as dist
    from torch_blocksparse_b200 import SparseSelfAttention, shard
    shards = shard.plan(Z, HEADS, world)
    s = shards[rank]
    c = problem_entries(args.attention, list(range(s.z0, s.z1)), s.h0, s.h1)
    in_bytes = 4 * c['q'].numel() * 2
    n_sets = max(1, min(8, math.ceil(400e6 / in_bytes)))
    mod = SparseSelfAttention(layout=c['layout'], block=c['block'], fused=True)
    step, state = make_steps(mod, c, dev, n_sets)
    # per-kernel durations come from a short run of their own, in which the backward is issued
    # kernel by kernel between events; the timed run issues it as the one call a user makes
    # (there the dQ kernel runs beside the dK / dV kernel on a second stream)
    prof, per_step_kernels = [], None
    if profile:
        _, prof = T.run(step, max(3, args.steps // 4), warmup=max(args.warmup, 3), profile=True)
        per_step_kernels = sum(a.elapsed_time(b) for _, a, b in prof) * 1e-3 / max(3, args.steps // 4)
    attempts = 0
    if sampler is not None:
        sampler.start()
    while True:                     # a run that took longer than its kernels issued one by one was disturbed from
        attempts += 1               # outside (the box is shared): it is taken again, at most twice
        elapsed, _ = T.run(state['graphed'], args.steps, warmup=max(args.warmup, 3), profile=False)
        busy = per_step_kernels * args.steps if profile else elapsed
        again = 1 if (profile and world == 1 and elapsed > 1.1 * busy and attempts < 3) else 0
        if not again:
            break
    clocks = sampler.stop() if sampler is not None else None
    eager, _ = T.run(step, args.steps, warmup=3, profile=False)          # the same steps issued call by call through autograd
    flops_total = workloads.attention_flops(c['full_layout'], c['block'], Z, HEAD_DIM)
    out = {'elapsed': elapsed, 'flops_total': flops_total, 'prof': prof, 'attempts': attempts, 'n_sets': n_sets,
           'shard': c, 'mod': mod, 'shards': shards, 'state': state, 'busy': busy,
           'local_shape': [s.z1 - s.z0, s.h1 - s.h0], 'clocks': clocks, 'eager': eager}
    if world > 1:
        state['graphed'](0)
        full = [shard.gather_dense(t.detach(), shards, Z, HEADS) for t in state['last']]
        digest = [float(t.double().sum()) for t in full]
        if rank == 0:
            # the sets rotate, but every set holds the same values: the last step's results are the problem's
            picks = [(Z - 1, HEADS - 1), (0, 5)][:n_slices_checked]
            entries = {z: workloads.config4(args.attention, Z=1, seed=z) for z in {z for z, _ in picks}}
            err = oracle_check(full, entries, picks)
            out['verify'] = {'gathered': 'o, dq, dk, dv all-gathered over NCCL into [%d, %d, %d, %d] tensors' % (Z, HEADS, SEQ, HEAD_DIM),
                             'oracle_slices': picks, 'max_err_over_tolerance': err, 'ok': bool(err <= 1.0),
                             'digest': digest}
        del full
    return out


def run_ours(args):
    import torch.distributed as dist
    from torch_blocksparse_b200 import SparseSelfAttention, fused, shard
    rank, world, local = dist_env()
    if not torch.cuda.is_available():
        raise SystemExit('bench.py needs a CUDA device (there is no CPU code path)')
    torch.cuda.set_device(local)
    dev = torch.device('cuda', local)
    if world > 1:
        os.environ.setdefault('MASTER_ADDR', '127.0.0.1')
        dist.init_process_group('nccl', device_id=dev)
    pk = peaks()
    T = Timing(dev, world)
    if args.only_matmul:
        if rank == 0:
            print(json.dumps({'matmul': matmul_bench(dev, pk, iters=max(1, args.steps), z=args.z, section=args.matmul_section)}))
        return
    if args.only_softmax:
        if rank == 0:
            print(json.dumps({'softmax': softmax_bench(dev, pk, iters=max(1, args.steps))}))
        return

    from torch_blocksparse_b200.host import bind_near_gpu
    numa_node = bind_near_gpu(dev)          # before any pinned allocation: host buffers local to the GPU
    Z = args.z
    main = run_sharded(args, T, dev, rank, world, Z, pk, profile=True, sampler=ClockSampler(local) if rank == 0 else None)
    clocks = main['clocks']
    elapsed, prof, c = main['elapsed'], main['prof'], main['shard']
    value = main['flops_total'] * args.steps / elapsed / 1e12
    Zl, Hl = main['local_shape']
    layout_l, block = c['layout'], c['block']

    # per-kernel durations inside the timed region (this rank's shard)
    kern = {}
    for name, a, b in prof:
        kern.setdefault(name, []).append(a.elapsed_time(b))
    kern_ms = {n: sum(t) / len(t) for n, t in kern.items()}
    top = max(kern_ms, key=kern_ms.get)
    per_product = 2 * Zl * int(layout_l.sum()) * block * block * HEAD_DIM
    counted = {'attn_fwd': 2, 'attn_bwd_dkdv': 2, 'attn_bwd_dq': 1, 'attn_bwd_delta': 0, 'attn_bwd_fused': 3}
    executed = {'attn_fwd': 2, 'attn_bwd_dkdv': 4, 'attn_bwd_dq': 3, 'attn_bwd_delta': 0, 'attn_bwd_fused': 5}
    achieved = counted[top] * per_product / (kern_ms[top] * 1e-3) / 1e12
    traffic = NCU_TRAFFIC_BYTES_PER_Z.get(top)
    roofline = {'bound': 'tensor', 'achieved': achieved, 'peak': pk['bf16_tflops'], 'unit': UNIT,
                'frac': achieved / pk['bf16_tflops'],
                'traffic': traffic * Zl * Hl / HEADS if traffic else None, 'kernel': top,
                'flops_counted_per_launch': counted[top] * per_product,
                'executed_tflops': executed[top] * per_product / (kern_ms[top] * 1e-3) / 1e12,
                'frac_of_sustained_peak': achieved / pk.get('bf16_tflops_sustained', pk['bf16_tflops']),
                'peak_source': pk['source'] + ' (bf16 dense, burst: the timed region lasts tens of milliseconds)'}

    # end to end: host -> device inputs and device -> host results inside the timed region,
    # through the library's host-operand entry (batch slices streamed over three CUDA streams)
    from torch_blocksparse_b200 import HostAttention
    mod = main['mod']
    host = {n: c[n].pin_memory() for n in ('q', 'k', 'v', 'do')}
    outs = [torch.empty_like(host['q']).pin_memory() for _ in range(4)]
    pipe = HostAttention(mod, Hl, SEQ, HEAD_DIM, c['q'].dtype, dev, slice_batch=1, depth=3)
    ins = [host[n] for n in ('q', 'k', 'v', 'do')]
    e2e_steps = max(3, min(args.steps, 10))
    pipe.run(*ins, *outs).synchronize()
    T.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(e2e_steps):
        done = pipe.run(*ins, *outs)
    torch.cuda.current_stream().wait_event(done)     # the last results are in host memory
    e1.record()
    T.barrier()
    e2e_t = T.max_over_ranks(e0.elapsed_time(e1) * 1e-3)
    pipe.check()                                     # (off the clock) no bounded device-side wait expired
    tensor_bytes = host['q'].numel() * host['q'].element_size()
    e2e = {'value': main['flops_total'] * e2e_steps / e2e_t / 1e12, 'unit': UNIT,
           'h2d_bytes_per_step': 4 * tensor_bytes * world, 'd2h_bytes_per_step': 4 * tensor_bytes * world,
           'ms_per_step': e2e_t / e2e_steps * 1e3, 'steps': e2e_steps, 'numa_node': numa_node,
           'host_copy_gbs_per_gpu_per_direction': 4 * tensor_bytes * e2e_steps / e2e_t / 1e9}
    del pipe, outs, host, ins

    extra = {}
    if world > 1 and not args.no_secondary:
        # every batch entry split over the heads of two ranks: layout slices and re-based tables on GPUs
        zs = max(1, world // 2)
        hs = run_sharded(args, T, dev, rank, world, zs, pk, profile=False, n_slices_checked=1)
        extra['head_split'] = {'workload': 'the same layout with Z=%d: every batch entry split over the heads of %d ranks'
                                           % (zs, world // zs),
                               'local_shape_z_h': hs['local_shape'], 'ms_per_step': hs['elapsed'] / args.steps * 1e3,
                               'tflops': hs['flops_total'] * args.steps / hs['elapsed'] / 1e12,
                               'verify': hs.get('verify')}
        del hs
        torch.cuda.empty_cache()
        # weak scaling: every rank a whole Z = Z_TOTAL problem of its own (entries rank*Z .. rank*Z + Z - 1)
        cw = problem_entries(args.attention, list(range(rank * Z, rank * Z + Z)))
        modw = SparseSelfAttention(layout=cw['layout'], block=cw['block'], fused=True)
        _, statew = make_steps(modw, cw, dev, 1)
        tw, _ = T.run(statew['graphed'], args.steps, warmup=3)
        extra['weak'] = {'workload': 'one full Z=%d problem per rank' % Z, 'ms_per_step': tw / args.steps * 1e3,
                         'tflops': workloads.attention_flops(cw['layout'], cw['block'], Z, HEAD_DIM) * world * args.steps / tw / 1e12}
        del cw, modw, statew

    if rank == 0:
        line = {
            'metric': METRIC, 'value': value, 'unit': UNIT, 'n_gpus': world, 'steps': args.steps,
            'warmup': max(args.warmup, 3), 'ms_per_step': elapsed / args.steps * 1e3, 'higher_is_better': True,
            'scaling': 'strong', 'vs_baseline': None, 'dtype': 'f16', 'data': 'synthetic',
            'config': config_dict(args, world, main['n_sets']), 'clocks': clocks, 'e2e': e2e,
            'gpu_launches': args.steps * (fused.KERNELS_PER_FWD + fused.KERNELS_PER_BWD),
            'roofline': roofline, 'kernel_ms': kern_ms, 'attempts': main['attempts'],
            'shard_z_h': main['local_shape'],
            'step_vs_kernels': {'kernels_one_by_one_ms_per_step': main['busy'] / args.steps * 1e3,
                                'elapsed_ms_per_step': elapsed / args.steps * 1e3,
                                'eager_ms_per_step': main['eager'] / args.steps * 1e3,
                                'note': 'the timed step replays forward + backward captured in a CUDA graph (SparseSelfAttention.graphed); '
                                        'eager = module(q, k, v).backward(do) call by call; in both the dQ kernel runs beside the '
                                        'dK / dV kernel on a second stream'},
            'frac_of_nominal_fp16_peak': value / world / 2250.0,
            'frac_of_measured_peak': value / world / pk['bf16_tflops'],
        }
        if Z != Z_TOTAL:
            line['reduced_workload'] = 'Z=%d instead of %d: not the headline configuration' % (Z, Z_TOTAL)
        if 'verify' in main:
            line['verify'] = main['verify']
        line.update(extra)
    del main
    torch.cuda.empty_cache()
    if rank == 0:
        if not args.no_cpu_baseline and world == 1:          # the host cores are timed on one rank at N = 1 only
            torch.set_num_threads(os.cpu_count() or 1)
            dt, fl = cpu_attention_sample(args.attention, args.cpu_slices)
            line['cpu_baseline'] = {'value': fl / dt / 1e12, 'unit': UNIT, 'cores': torch.get_num_threads(), 'kind': 'port',
                                    'sample': '%d of the %d (batch, head) slices, dense-masked FP32 torch on FP16-rounded '
                                              'inputs, %.1f s' % (args.cpu_slices, Z_TOTAL * HEADS, dt)}
        if world == 1 and not args.no_extras:
            T1 = Timing(dev, 1)
            other = 'bidirectional' if args.attention == 'unidirectional' else 'unidirectional'
            cb = problem_entries(other, list(range(Z)))
            line['config4_' + other] = attention_section('config4 %s, FP16, Z=%d' % (other, Z), cb, dev,
                                                         max(3, args.steps // 2), pk, T1, 'f16')
            del cb
            torch.cuda.empty_cache()
            # configuration 4 called with configuration 3's optional inputs: a relative position bias
            # (broadcast over the batch), a key-padding mask ('add', -inf) and a causal 'mul' mask
            cm = problem_entries(args.attention, list(range(Z)))
            gm = torch.Generator(device=dev).manual_seed(3)
            rpe = 0.1 * torch.randn((HEADS, SEQ, SEQ), generator=gm, device=dev, dtype=torch.float16)
            lengths = torch.randint(SEQ // 2, SEQ + 1, (Z,), generator=torch.Generator().manual_seed(3))
            kpm = torch.zeros((Z, SEQ), dtype=torch.float16)
            kpm[torch.arange(SEQ)[None, :] >= lengths[:, None]] = float('-inf')
            sec = attention_section('config4 %s, FP16, Z=%d, with rpe [H, L, L], key-padding mask and causal mask'
                                    % (args.attention, Z), cm, dev, max(3, args.steps // 2), pk, T1, 'f16',
                                    rpe=rpe, key_padding_mask=kpm.to(dev),
                                    attn_mask=torch.tril(torch.ones((SEQ, SEQ), dtype=torch.float16, device=dev)))
            sec['ratio_to_plain_step'] = sec['ms_per_step'] / line['ms_per_step']
            line['config4_with_config3_inputs'] = sec
            del cm, rpe, kpm
            torch.cuda.empty_cache()
            # configuration 5 at its full size on one GPU (17 GB of operands and results); the inputs
            # are drawn on the device (the CPU generator needs a minute for 4 x 1 G values)
            c5 = workloads.config5(small=False, Z=1)
            g = torch.Generator(device=dev).manual_seed(0)
            shape = (32,) + tuple(c5['q'].shape[1:])
            for n in ('q', 'k', 'v', 'do'):
                c5[n] = torch.randn(shape, generator=g, device=dev, dtype=torch.bfloat16)
            line['config5'] = attention_section('config5: BigBird-style BF16, Z=32, H=16, L=16384, head_dim 128, block 128 '
                                                '(all of it on one GPU)', c5, dev, 3, pk, T1, 'bf16')
            del c5
            torch.cuda.empty_cache()
        if world == 1 and not args.no_softmax:
            line['softmax'] = softmax_bench(dev, pk)
        if world == 1 and not args.no_extras:
            line['matmul'] = matmul_bench(dev, pk, iters=5)
            line['table_build'] = table_build_times(dev)
        print(json.dumps(line))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument('--gpus', type=int, default=1)
    ap.add_argument('--steps', type=int, default=20)
    ap.add_argument('--warmup', type=int, default=5)
    ap.add_argument('--impl', default='ours', choices=['ours', 'reference'])
    ap.add_argument('--attention', default='unidirectional', choices=['unidirectional', 'bidirectional'])
    ap.add_argument('--cpu-slices', type=int, default=16, help='(batch, head) slices timed for cpu_baseline')
    ap.add_argument('--ref-slices', type=int, default=16, help='(batch, head) slices per step of --impl reference')
    ap.add_argument('--no-softmax', action='store_true')
    ap.add_argument('--no-extras', action='store_true', help='skip the other configurations (C4 bidirectional, C5, MatMul)')
    ap.add_argument('--no-secondary', action='store_true', help='N > 1: skip the head-split and weak-scaling runs')
    ap.add_argument('--only-softmax', action='store_true', help='run only the softmax section (profiling aid)')
    ap.add_argument('--only-matmul', action='store_true', help='run only the MatMul section')
    ap.add_argument('--matmul-section', choices=['all', 'config2', 'large'], default='all',
                    help='with --only-matmul: configuration 1 + 2 only, or blocks 64 / 128 only (profiling aid)')
    ap.add_argument('--z', type=int, default=Z_TOTAL, help='batch entries of the problem; anything but 8 is a reduced, '
                    'non-headline workload (profiling aid) and is flagged in the output')
    ap.add_argument('--no-cpu-baseline', action='store_true')
    args = ap.parse_args()
    if args.impl == 'reference':
        run_reference(args)
    else:
        run_ours(args)


if __name__ == '__main__':
    main()
