"""Benchmark of the block-sparse attention hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload (config.workload): sparse self-attention forward + backward, FP16,
Z=8 per GPU, H=16, L=8192, head_dim 64, block 64, "fixed" layout (local windows
of 4 blocks, last block of every window global, unidirectional) -- the
configuration the headline metric is quoted on.  Inputs are seeded synthetic
N(0,1) tensors of that shape (the reference measures on no dataset).

One "step" is one forward + backward through the public wrapper
(SparseSelfAttention).  `value` counts only the FLOPs of nonzero blocks
(6 products of 2*Z*nnz*block^2*D; softmax and recomputation are not counted)
with inputs resident in HBM; `e2e` is the same step on operands in pinned host
memory through the library's host entry (HostAttention): every step copies its
inputs in and its four results out inside the timed region, streamed by batch
slices so that transfers and kernels overlap.
With N > 1 every rank runs the same-size shard of a Z = 8N batch (independent
(batch, head) units, no collective on the timed path: weak scaling); NCCL is
only used to reduce the timings and to all-gather outputs for verification.

`--impl reference` times the reference's dense-masked definition of the same
op on the host cores (the CPU restatement under oracle/), on a bounded sample
of (batch, head) slices.
"""
import argparse
import json
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

# dram__bytes_read.sum + dram__bytes_write.sum per launch from the ncu captures
# summarised under profiles/.  The attention figure was captured at Z=2 (225.8 MB)
# and scaled by 4 to the Z=8 launch: every (batch, head) pair is independent, so
# traffic grows in proportion.
NCU_TRAFFIC_BYTES = {'attn_bwd_dkdv': 4 * 225.8e6, 'softmax_fwd': 638.5e6, 'softmax_bwd': 924.3e6}


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


def cpu_attention_sample(c, n_slices, repeats=1):
    """Times the dense-masked CPU definition on `n_slices` (batch, head) slices of
    the workload.  Returns (seconds per pass over the sample, counted FLOPs of the sample)."""
    from oracle import dense_masked as dm
    layout, block = c['layout'], c['block']
    Z, H = c['q'].shape[:2]
    slices = [(i % Z, (i * 7) % H) for i in range(n_slices)]
    flops = 0
    for z, h in slices:
        flops += workloads.attention_flops(layout[h:h + 1], block, 1, c['q'].size(-1))
    best = None
    for _ in range(repeats):
        t0 = time.perf_counter()
        for z, h in slices:
            dm.attention_reference(c['q'][z:z + 1, h:h + 1], c['k'][z:z + 1, h:h + 1], c['v'][z:z + 1, h:h + 1],
                                   layout[h:h + 1], block, c['scale'], do=c['do'][z:z + 1, h:h + 1])
        dt = time.perf_counter() - t0
        best = dt if best is None else min(best, dt)
    return best, flops


def run_reference(args):
    rank, world, _ = dist_env()
    if rank != 0:
        return
    torch.set_num_threads(os.cpu_count() or 1)
    c = workloads.config4(args.attention, Z=1)
    n_slices = args.ref_slices
    for _ in range(args.warmup):
        cpu_attention_sample(c, n_slices)
    t0 = time.perf_counter()
    flops = 0
    for _ in range(args.steps):
        _, f = cpu_attention_sample(c, n_slices)
        flops += f
    dt = time.perf_counter() - t0
    value = flops / dt / 1e12
    sample = ('%d of the %d (batch, head) slices per step, dense-masked FP32 torch on FP16-rounded inputs'
              % (n_slices, 8 * 16 * max(1, args.gpus)))
    line = {
        'impl': 'reference', 'metric': METRIC, 'value': value, 'unit': UNIT, 'n_gpus': args.gpus,
        'steps': args.steps, 'warmup': args.warmup, 'ms_per_step': dt / args.steps * 1e3,
        'higher_is_better': True, 'scaling': 'weak', 'vs_baseline': None, 'dtype': 'f32', 'data': 'synthetic',
        'config': config_dict(args, world),
        'cpu_baseline': {'value': value, 'unit': UNIT, 'cores': torch.get_num_threads(), 'kind': 'port', 'sample': sample},
        'e2e': {'value': value, 'unit': UNIT, 'h2d_bytes_per_step': 0, 'd2h_bytes_per_step': 0},
        'gpu_launches': 0,
    }
    print(json.dumps(line))


def config_dict(args, world):
    return {'workload': 'config4: sparse self-attention fwd+bwd FP16, Z=8 per GPU, H=16, L=8192, head_dim=64, '
                        'block=64, fixed layout (windows of 4 blocks, last block global), %s' % args.attention,
            'global_batch': 8 * world, 'seq_len': 8192, 'heads': 16, 'head_dim': 64, 'block': 64,
            'parallelism': '(batch, head) shards, one per GPU, no collective',
            'l2': 'inputs (4 x 134 MB per GPU) exceed the 126 MB L2; no explicit flush'}


def matmul_bench(dev, pk, iters=10, z=8):
    """Block-sparse MatMul (configuration 2: dsd / dds, FP16, block 32, Z=8, H=8, 2048^3, layout
    Bernoulli(0.25)), forward and forward + backward, TFLOP/s on nonzero-block FLOPs."""
    from torch_blocksparse_b200 import MatMul
    out = {'workload': 'config2: dsd / dds FP16, block 32, Z=%d, H=8, M=N=K=2048, Bernoulli(0.25) layout' % z, 'cases': []}
    peak_tf = pk.get('bf16_tflops_sustained', pk['bf16_tflops'])

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
    return out


def softmax_bench(dev, pk, iters=20):
    """Sparse softmax (configuration 3) forward / backward bandwidth."""
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
    tf, tb = timeit(fwd), timeit(bwd)
    return {
        'workload': 'config3: FP16, block 64, Z=8, H=16, 4096x4096, causal band of 4 + first column, scale, rpe, '
                    'key-padding mask (add), causal mask (mul)',
        'fwd_gbs': fwd_bytes / tf / 1e9, 'bwd_gbs': bwd_bytes / tb / 1e9,
        'fwd_ms': tf * 1e3, 'bwd_ms': tb * 1e3, 'fwd_bytes': fwd_bytes, 'bwd_bytes': bwd_bytes,
        'roofline': {'bound': 'hbm', 'achieved': fwd_bytes / tf / 1e9, 'peak': pk['hbm_gbs'], 'unit': 'GB/s',
                     'frac': fwd_bytes / tf / 1e9 / pk['hbm_gbs'], 'traffic': NCU_TRAFFIC_BYTES['softmax_fwd'],
                     'kernel': 'softmax_fwd_zloop', 'peak_source': pk['source']},
        'roofline_bwd': {'bound': 'hbm', 'achieved': bwd_bytes / tb / 1e9, 'peak': pk['hbm_gbs'], 'unit': 'GB/s',
                         'frac': bwd_bytes / tb / 1e9 / pk['hbm_gbs'], 'traffic': NCU_TRAFFIC_BYTES['softmax_bwd'],
                         'kernel': 'softmax_bwd_group', 'peak_source': pk['source']},
        'gpu_launches': 2 * (iters + 3),
    }


def run_ours(args):
    import torch.distributed as dist
    from torch_blocksparse_b200 import SparseSelfAttention, fused
    rank, world, local = dist_env()
    if not torch.cuda.is_available():
        raise SystemExit('bench.py needs a CUDA device (there is no CPU code path)')
    torch.cuda.set_device(local)
    dev = torch.device('cuda', local)
    if world > 1:
        os.environ.setdefault('MASTER_ADDR', '127.0.0.1')
        dist.init_process_group('nccl', device_id=dev)
    pk = peaks()
    if args.only_matmul:
        if rank == 0:
            print(json.dumps({'matmul': matmul_bench(dev, pk, iters=max(1, args.steps), z=args.z)}))
        return
    if args.only_softmax:
        if rank == 0:
            print(json.dumps({'softmax': softmax_bench(dev, pk, iters=max(1, args.steps))}))
        return

    from torch_blocksparse_b200.host import bind_near_gpu
    numa_node = bind_near_gpu(dev)          # before any pinned allocation: host buffers local to the GPU
    c = workloads.config4(args.attention, Z=args.z, seed=rank)
    layout, block, D = c['layout'], c['block'], c['q'].size(-1)
    Z = c['q'].size(0)
    flops_step = workloads.attention_flops(layout, block, Z, D)       # this rank's shard
    mod = SparseSelfAttention(layout=layout, block=block, fused=True)
    host = {n: c[n].pin_memory() for n in ('q', 'k', 'v', 'do')}
    q, k, v = (host[n].to(dev).requires_grad_() for n in ('q', 'k', 'v'))
    do = host['do'].to(dev)

    def step():
        q.grad = k.grad = v.grad = None
        o = mod(q, k, v)
        o.backward(do)
        return o

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed_steps():
        """K steps between two events on the current stream, barrier + synchronize on both
        sides, max over ranks.  Returns (seconds, per-kernel event triples)."""
        fused.PROFILE = []
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        t0.record()
        for _ in range(args.steps):
            step()
        t1.record()
        barrier()
        prof, fused.PROFILE = fused.PROFILE, None
        el = torch.tensor([t0.elapsed_time(t1) * 1e-3], device=dev, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(el, op=dist.ReduceOp.MAX)
        return float(el), prof

    fused.PROFILE = []                      # warm up on the code path that is timed
    for _ in range(max(args.warmup, 3)):
        step()
    fused.PROFILE = None
    barrier()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    # A measurement in which the kernels account for less than 90 % of the elapsed time was
    # disturbed from outside the kernels (the box is shared); it is taken again, at most twice.
    attempts = 0
    while True:
        attempts += 1
        elapsed, prof = timed_steps()
        busy = sum(a.elapsed_time(b) for _, a, b in prof) * 1e-3
        retry = torch.tensor([1 if (busy < 0.9 * elapsed and attempts < 3) else 0], device=dev)
        if world > 1:
            dist.all_reduce(retry, op=dist.ReduceOp.MAX)
        if not int(retry):
            break
    clocks = sampler.stop() if rank == 0 else None
    value = flops_step * world * args.steps / elapsed / 1e12

    # per-kernel durations inside the timed region
    kern = {}
    for name, a, b in prof:
        kern.setdefault(name, []).append(a.elapsed_time(b))
    kern_ms = {n: sum(t) / len(t) for n, t in kern.items()}
    top = max(kern_ms, key=kern_ms.get)
    per_product = 2 * Z * int(layout.sum()) * block * block * D
    counted = {'attn_fwd': 2, 'attn_bwd_dkdv': 2, 'attn_bwd_dq': 1, 'attn_bwd_delta': 0}
    executed = {'attn_fwd': 2, 'attn_bwd_dkdv': 4, 'attn_bwd_dq': 3, 'attn_bwd_delta': 0}
    peak_tf = pk.get('bf16_tflops_sustained', pk['bf16_tflops'])
    achieved = counted[top] * per_product / (kern_ms[top] * 1e-3) / 1e12
    roofline = {'bound': 'tensor', 'achieved': achieved, 'peak': peak_tf, 'unit': 'TFLOP/s', 'frac': achieved / peak_tf,
                'traffic': NCU_TRAFFIC_BYTES.get(top), 'kernel': top,
                'flops_counted_per_launch': counted[top] * per_product,
                'executed_tflops': executed[top] * per_product / (kern_ms[top] * 1e-3) / 1e12,
                'peak_source': pk['source'] + ' (bf16 dense, sustained)'}

    # end to end: host -> device inputs and device -> host results inside the timed region,
    # through the library's host-operand entry (batch slices streamed over three CUDA streams)
    from torch_blocksparse_b200 import HostAttention
    outs = [torch.empty_like(host['q']).pin_memory() for _ in range(4)]
    pipe = HostAttention(mod, c['q'].size(1), c['q'].size(2), D, c['q'].dtype, dev, slice_batch=1, depth=3)
    ins = [host[n] for n in ('q', 'k', 'v', 'do')]

    def e2e_step():
        return pipe.run(*ins, *outs)

    e2e_steps = max(3, min(args.steps, 10))
    e2e_step().synchronize()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(e2e_steps):
        done = e2e_step()
    torch.cuda.current_stream().wait_event(done)     # the last results are in host memory
    e1.record()
    barrier()
    e2e_t = torch.tensor([e0.elapsed_time(e1) * 1e-3], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(e2e_t, op=dist.ReduceOp.MAX)
    tensor_bytes = host['q'].numel() * host['q'].element_size()
    e2e = {'value': flops_step * world * e2e_steps / float(e2e_t) / 1e12, 'unit': UNIT,
           'h2d_bytes_per_step': 4 * tensor_bytes, 'd2h_bytes_per_step': 4 * tensor_bytes,
           'ms_per_step': float(e2e_t) / e2e_steps * 1e3, 'steps': e2e_steps, 'numa_node': numa_node}

    # verification off the clock: all-gather a digest of every rank's outputs, and
    # have rank 0 recompute the last rank's shard and compare bit for bit
    verify = None
    if world > 1:
        o = step()
        digest = torch.stack([t.double().sum() for t in (o.detach(), q.grad, k.grad, v.grad)])
        parts = [torch.empty_like(digest) for _ in range(world)]
        dist.all_gather(parts, digest)
        if rank == 0:
            other = workloads.config4(args.attention, Z=args.z, seed=world - 1)
            q2, k2, v2 = (other[n].to(dev).requires_grad_() for n in ('q', 'k', 'v'))
            o2 = mod(q2, k2, v2)
            o2.backward(other['do'].to(dev))
            mine = torch.stack([t.double().sum() for t in (o2.detach(), q2.grad, k2.grad, v2.grad)])
            verify = {'gathered_ranks': world, 'recomputed_rank': world - 1,
                      'digest_equal': bool(torch.equal(mine, parts[world - 1]))}

    if rank == 0:
        line = {
            'metric': METRIC, 'value': value, 'unit': UNIT, 'n_gpus': world, 'steps': args.steps,
            'warmup': max(args.warmup, 3), 'ms_per_step': elapsed / args.steps * 1e3, 'higher_is_better': True,
            'scaling': 'weak', 'vs_baseline': None, 'dtype': 'f16', 'data': 'synthetic',
            'config': config_dict(args, world), 'clocks': clocks, 'e2e': e2e,
            'gpu_launches': args.steps * (fused.KERNELS_PER_FWD + fused.KERNELS_PER_BWD),
            'roofline': roofline, 'kernel_ms': kern_ms, 'attempts': attempts,
            'frac_of_nominal_fp16_peak': value / world / 2250.0,
            'frac_of_measured_peak': value / world / peak_tf,
        }
        if args.z != 8:
            line['reduced_workload'] = 'Z=%d per GPU instead of 8: not the headline configuration' % args.z
        if not args.no_cpu_baseline and world == 1:          # the host cores are timed on one rank at N = 1 only
            torch.set_num_threads(os.cpu_count() or 1)
            dt, fl = cpu_attention_sample(c, args.cpu_slices)
            line['cpu_baseline'] = {'value': fl / dt / 1e12, 'unit': UNIT, 'cores': torch.get_num_threads(), 'kind': 'port',
                                    'sample': '%d of the %d (batch, head) slices, dense-masked FP32 torch on FP16-rounded '
                                              'inputs, %.1f s' % (args.cpu_slices, Z * 16 * world, dt)}
        if not args.no_softmax:
            line['softmax'] = softmax_bench(dev, pk)
        if verify is not None:
            line['verify'] = verify
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
    ap.add_argument('--ref-slices', type=int, default=2, help='(batch, head) slices per step of --impl reference')
    ap.add_argument('--no-softmax', action='store_true')
    ap.add_argument('--only-softmax', action='store_true', help='run only the softmax section (profiling aid)')
    ap.add_argument('--only-matmul', action='store_true', help='run only the MatMul section (configuration 2)')
    ap.add_argument('--z', type=int, default=8, help='batch entries per GPU; anything but 8 is a reduced, '
                    'non-headline workload (profiling aid) and is flagged in the output')
    ap.add_argument('--no-cpu-baseline', action='store_true')
    args = ap.parse_args()
    if args.impl == 'reference':
        run_reference(args)
    else:
        run_ours(args)


if __name__ == '__main__':
    main()
