"""Sparse self-attention forward + backward for operands that live in host memory.

The reference has no such entry: its ops take device tensors and a caller with
host data copies everything in, runs, and copies everything out, one after the
other (torch_blocksparse/deepspeedsparseselfattention.py:135-166 sees device
tensors only).  Every (batch, head) pair of this path is independent, so the
work is streamed by batch slices instead: three CUDA streams (host -> device,
kernels, device -> host) run as a pipeline over a small ring of device-side
slice buffers, and a step costs about the larger of the two PCIe transfers
instead of their sum plus the kernels.

    pipe = HostAttention(module, heads, length, head_dim, dtype, device)
    done = pipe.run(q, k, v, do, o, dq, dk, dv)      # pinned host tensors [Z, H, L, D]
    done.synchronize()                               # or torch.cuda.current_stream().wait_event(done)

Successive run() calls queue behind each other on the three streams, so the
copies of one call overlap the kernels and the read-back of the previous one.
Only the unmasked case (no rpe / masks) is offered here.
"""
import torch

from . import _lib
from .matmul import _dtype_code


def _cpus_near_gpu(device):
    """(NUMA node or None, set of CPUs next to the GPU or None), from sysfs, else from NVML
    (read-only queries).  Containers often hide the PCI tree of sysfs; NVML still answers."""
    p = torch.cuda.get_device_properties(device)
    bdf = '%04x:%02x:%02x.0' % (p.pci_domain_id, p.pci_bus_id, p.pci_device_id)
    try:
        with open('/sys/bus/pci/devices/%s/numa_node' % bdf) as f:
            node = int(f.read())
        if node >= 0:
            with open('/sys/devices/system/node/node%d/cpulist' % node) as f:
                cpus = set()
                for part in f.read().strip().split(','):
                    lo, _, hi = part.partition('-')
                    cpus.update(range(int(lo), int(hi or lo) + 1))
            return node, cpus
    except (OSError, ValueError):
        pass
    try:
        import os
        import pynvml
        pynvml.nvmlInit()
        try:
            h = pynvml.nvmlDeviceGetHandleByPciBusId(('0000' + bdf).encode())
            words = (max(os.sched_getaffinity(0)) + 64) // 64 + 16
            mask = pynvml.nvmlDeviceGetCpuAffinity(h, words)
            cpus = {64 * w + b for w, m in enumerate(mask) for b in range(64) if (int(m) >> b) & 1}
            node = None
            if hasattr(pynvml, 'nvmlDeviceGetNumaNodeId'):
                try:
                    node = int(pynvml.nvmlDeviceGetNumaNodeId(h))
                except pynvml.NVMLError:
                    node = None
            return node, (cpus or None)
        finally:
            pynvml.nvmlShutdown()
    except Exception:                        # no NVML, an older driver, a query it refuses
        return None, None


def bind_near_gpu(device):
    """Restricts the calling process to the CPU cores next to the GPU (its NUMA node), so that
    pinned buffers allocated afterwards (first touch) are local to the GPU's PCIe root.  With one
    process per GPU this keeps the host side of several concurrent pipelines off the inter-socket
    link.  Returns the node (or -1 when only the CPU set is known), or None when the topology
    cannot be read or none of those cores is available to this process (then nothing is
    changed).  Linux only."""
    import os
    try:
        node, cpus = _cpus_near_gpu(device)
        if not cpus:
            return None
        allowed = cpus & os.sched_getaffinity(0)
        if not allowed:
            return None
        os.sched_setaffinity(0, allowed)
        return -1 if node is None else node
    except (OSError, ValueError, AttributeError):
        return None


class HostAttention:

    def __init__(self, module, heads, length, head_dim, dtype=torch.float16, device='cuda',
                 slice_batch=1, depth=3):
        """module: a DeepSpeedSparseSelfAttention / SparseSelfAttention (its layout, block and tile
        lists are used); slice_batch: batch entries per pipeline slice; depth: slices in flight."""
        if dtype not in (torch.float16, torch.bfloat16):
            raise ValueError('host pipeline: FP16 or BF16 operands')
        if head_dim not in (64, 128):
            raise NotImplementedError('host pipeline: head dimensions 64 and 128')
        self.device = torch.device(device)
        if self.device.type != 'cuda':
            raise ValueError('host pipeline: a CUDA device is required')
        self.H, self.L, self.D, self.dtype = heads, length, head_dim, dtype
        self.block = module.block
        sdd_nt, _, _ = module.get_ops(heads, length)
        self.meta = sdd_nt.meta
        self.tiles = module.tiles.get((heads, length))
        self.zs, self.depth = slice_batch, depth
        shape = (slice_batch, heads, length, head_dim)
        with torch.cuda.device(self.device):
            self.streams = [torch.cuda.Stream() for _ in range(3)]        # in, kernels, out
            self.slots = []
            for _ in range(depth):
                t = {n: torch.empty(shape, dtype=dtype, device=self.device)
                     for n in ('q', 'k', 'v', 'do', 'o', 'dq', 'dk', 'dv')}
                t['lse'] = torch.empty(shape[:3], dtype=torch.float32, device=self.device)
                t['delta'] = torch.empty(shape[:3], dtype=torch.float32, device=self.device)
                t['ev'] = [torch.cuda.Event() for _ in range(3)]           # loaded, computed, drained
                t['used'] = False
                self.slots.append(t)

    def _check(self, name, x, Z):
        if x.is_cuda or not x.is_pinned():
            raise ValueError('host pipeline: %s must be a pinned host tensor' % name)
        if tuple(x.shape) != (Z, self.H, self.L, self.D) or x.dtype != self.dtype or not x.is_contiguous():
            raise ValueError('host pipeline: %s must be a contiguous %s tensor of shape [%d, %d, %d, %d]'
                             % (name, self.dtype, Z, self.H, self.L, self.D))

    def _kernels(self, t, z, scale, stream):
        L_ = _lib.lib()
        tiles = (self.tiles.hdr.data_ptr(), self.tiles.on(self.device).data_ptr()) if self.tiles is not None else (None, None)
        meta = (self.meta.hdr.data_ptr(), self.meta.on(self.device).data_ptr())
        st = t['q'].stride()
        strides = (st[0], st[1], st[2])
        none_masks = (None, 0, 0, 0, None, 0, 0, None, 0, 0)
        code = _dtype_code(t['q'])
        _lib.check(L_.bsp_attn_fwd(
            t['q'].data_ptr(), t['k'].data_ptr(), t['v'].data_ptr(), t['o'].data_ptr(), t['lse'].data_ptr(),
            code, self.block, z, self.H, self.L, self.D, *strides, *strides, *strides, *strides,
            *meta, *tiles, scale, *none_masks, stream))
        _lib.check(L_.bsp_attn_bwd(
            t['q'].data_ptr(), t['k'].data_ptr(), t['v'].data_ptr(), t['o'].data_ptr(), t['do'].data_ptr(),
            t['lse'].data_ptr(), t['delta'].data_ptr(), t['dq'].data_ptr(), t['dk'].data_ptr(), t['dv'].data_ptr(),
            code, self.block, z, self.H, self.L, self.D, *strides, *strides, *strides, *strides, *strides,
            *meta, *tiles, scale, *none_masks, stream))

    def check(self):
        """Waits for everything queued so far and raises RuntimeError if a bounded wait inside one of
        the kernels expired (the results of that run are then not valid)."""
        for s in self.streams:
            s.synchronize()
        _lib.check_device()

    def run(self, q, k, v, do, o, dq, dk, dv, scale=None):
        """Queues forward + backward for host operands q, k, v, do and host results o, dq, dk,
        dv.  Returns a CUDA event that completes when every result is in host memory."""
        Z = q.size(0)
        for name, x in (('q', q), ('k', k), ('v', v), ('do', do), ('o', o), ('dq', dq), ('dk', dk), ('dv', dv)):
            self._check(name, x, Z)
        scale = float(self.D) ** -0.5 if scale is None else float(scale)
        s_in, s_k, s_out = self.streams
        ins, outs = (('q', q), ('k', k), ('v', v), ('do', do)), (('o', o), ('dq', dq), ('dk', dk), ('dv', dv))
        with torch.cuda.device(self.device):
            start = torch.cuda.Event()
            start.record()                       # work queued by the caller before this call comes first
            s_in.wait_event(start)
            for i, z0 in enumerate(range(0, Z, self.zs)):
                z = min(self.zs, Z - z0)
                t = self.slots[i % self.depth]
                loaded, computed, drained = t['ev']
                with torch.cuda.stream(s_in):
                    if t['used']:
                        s_in.wait_event(drained)                    # the slot's last results have left
                    for n, h in ins:
                        t[n][:z].copy_(h[z0:z0 + z], non_blocking=True)
                    loaded.record()
                with torch.cuda.stream(s_k):
                    s_k.wait_event(loaded)
                    self._kernels(t, z, scale, s_k.cuda_stream)
                    computed.record()
                with torch.cuda.stream(s_out):
                    s_out.wait_event(computed)
                    for n, h in outs:
                        h[z0:z0 + z].copy_(t[n][:z], non_blocking=True)
                    drained.record()
                t['used'] = True
            done = torch.cuda.Event()
            done.record(s_out)
        return done
