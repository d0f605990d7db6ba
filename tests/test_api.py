"""Host-side behaviour of the Python interface: constructor arguments, error
types and the structure of the table tuples, as in the reference."""
import pytest
import torch

import torch_blocksparse_b200 as tbs
from torch_blocksparse_b200 import shard
from torch_blocksparse_b200.matmul import _sparse_matmul
from torch_blocksparse_b200.softmax import _sparse_softmax


def test_exports():
    for name in ('MatMul', 'Softmax', 'SparseSelfAttention', 'DeepSpeedSparseSelfAttention', 'SparsityConfig'):
        assert hasattr(tbs, name)
    assert tbs.SparseSelfAttention is tbs.DeepSpeedSparseSelfAttention


def test_matmul_constructor_and_attributes():
    layout = torch.ones((2, 4, 4), dtype=torch.long)
    with pytest.raises(NotImplementedError, match='Supported modes are: sdd, dsd, dds'):
        tbs.MatMul(layout, 16, 'ssd')
    op = tbs.MatMul(layout, 16, 'dsd', trans_a=True, bench=True)
    assert (op.trans_a, op.trans_b, op.mode, op.block, op.bench) == (True, False, 'dsd', 16, True)
    assert tuple(op.spdims) == (2, 4, 4) and op.layout is layout
    assert op.time_c is None and op.time_da is None and op.time_db is None and op.lut_cache == {}


@pytest.mark.parametrize('mode', ['sdd', 'dsd', 'dds'])
def test_make_lut_tuple_structure(mode):
    """(c, da, db) x (lut, num_locks, width, packs): an SDD entry is (list, None, list, list),
    a DSD/DDS entry (tensor, int, int, None) -- torch_blocksparse/matmul.py:611-641."""
    g = torch.Generator().manual_seed(0)
    layout = (torch.rand((2, 8, 8), generator=g) > 0.5).long()
    layout[:, 0, 0] = 1
    op = tbs.MatMul(layout, 16, mode, trans_a=(mode == 'dsd'))
    t = op.make_lut(torch.float16, 'cpu')
    assert len(t) == 12 and op.make_lut(torch.float16, 'cpu') is t
    which = {'sdd': 0, 'dsd': 1, 'dds': 2}[mode]
    for slot in range(3):
        lut, nlocks, width, packs = t[4 * slot:4 * slot + 4]
        if slot == which:
            assert isinstance(lut, list) and nlocks is None and isinstance(width, list) and isinstance(packs, list)
            assert sum(w * p * p for w, p in zip(width, packs)) == int(layout.sum())
        else:
            assert lut.dtype == torch.int32 and nlocks == 1 and packs is None
            assert lut.numel() == 6 * width + 2 * int(layout.sum()) + 2
    # FP32 halves the K step of the DSD/DDS tables (matmul.py:617)
    t32 = op.make_lut(torch.float32, 'cpu')
    slot = (which + 1) % 3
    assert t32[4 * slot].numel() == 6 * t32[4 * slot + 2] + 2 * int(layout.sum()) * 2 + 2
    # the static builders of the autograd class are callable as in the reference
    assert len(_sparse_matmul.make_sdd_lut(layout, 16, torch.float16, 'cpu')) == 4
    assert len(_sparse_matmul.make_dxx_lut(layout, 16, 16, True, 'cpu')) == 4


def test_softmax_constructor_and_dtype_errors():
    layout = torch.ones((1, 2, 2), dtype=torch.long)
    op = tbs.Softmax(layout, 16)
    assert tuple(op.spdims) == (1, 2, 2) and op.block == 16 and op.bench is False and op.lut_cache == {}
    lut, maxlut = op.make_lut(torch.device('cpu'))
    assert maxlut == 2 and lut.numel() == 2 * 2 + 4 * 4
    assert _sparse_softmax.make_lut(layout, 16, 'cpu')[1] == 2
    x = torch.zeros((1, 4, 16, 16), dtype=torch.float16)
    with pytest.raises(ValueError, match='relative position embedding'):
        op(x, rpe=torch.zeros((1, 1, 32, 32)))
    with pytest.raises(ValueError, match='Attention mask'):
        op(x, attn_mask=torch.zeros((32, 32)))
    with pytest.raises(ValueError, match='Key padding mask'):
        op(x, key_padding_mask=torch.zeros((1, 32)))


def test_no_cpu_code_path():
    layout = torch.ones((1, 2, 2), dtype=torch.long)
    with pytest.raises(RuntimeError, match='CUDA tensors only'):
        tbs.Softmax(layout, 16)(torch.zeros((1, 4, 16, 16)))
    with pytest.raises(RuntimeError, match='CUDA tensors only'):
        tbs.MatMul(layout, 16, 'sdd')(torch.zeros((1, 1, 32, 16)), torch.zeros((1, 1, 16, 32)))
    with pytest.raises(RuntimeError, match='CUDA tensors only'):
        q = torch.zeros((1, 1, 32, 64), dtype=torch.float16)
        tbs.SparseSelfAttention(layout=layout, block=16)(q, q, q)


def test_sparsity_config_and_wrapper_errors():
    with pytest.raises(NotImplementedError):
        tbs.SparsityConfig(mode='variable')
    with pytest.raises(NotImplementedError):
        tbs.SparsityConfig(attention='causal')
    cfg = tbs.SparsityConfig(mode='fixed', block=64, stride=256)
    mod = tbs.DeepSpeedSparseSelfAttention(cfg)
    assert (mod.key_padding_mask_mode, mod.attn_mask_mode) == ('add', 'mul')
    lay = mod.get_layout(16, 8192)
    assert tuple(lay.shape) == (16, 128, 128) and int(lay.sum()) == 36864
    with pytest.raises(ValueError):
        mod.get_layout(16, 8200)
    with pytest.raises(ValueError):
        tbs.DeepSpeedSparseSelfAttention(tbs.SparsityConfig(block=64, stride=96)).get_layout(2, 1024)
    with pytest.raises(ValueError):
        tbs.SparseSelfAttention(layout=torch.ones((2, 4, 4), dtype=torch.long))
    q = torch.zeros((1, 2, 64, 64))
    with pytest.raises(NotImplementedError, match='only self-attention'):
        tbs.SparseSelfAttention(layout=torch.ones((2, 4, 4), dtype=torch.long), block=16)(q, q[:, :, :32], q)
    # two modules with different layouts and equal length keep separate op caches
    a = tbs.SparseSelfAttention(layout=torch.ones((2, 4, 4), dtype=torch.long), block=16)
    b = tbs.SparseSelfAttention(layout=torch.eye(4, dtype=torch.long)[None].repeat(2, 1, 1), block=16)
    assert a.get_ops(2, 64)[0].layout.sum() != b.get_ops(2, 64)[0].layout.sum()


def test_layout_generators():
    lay = tbs.layouts.causal_band(16, 64, 4, 1)
    assert int(lay.sum()) == 4960 and int(lay[0].sum(1).max()) == 5
    bb = tbs.layouts.bigbird(16, 128, 3, 3, 2, seed=0)
    assert tuple(bb.shape) == (16, 128, 128) and bool((bb[:, :2] == 1).all()) and bool((bb[:, :, :2] == 1).all())
    assert torch.equal(bb, tbs.layouts.bigbird(16, 128, 3, 3, 2, seed=0))
    assert int(tbs.layouts.fixed(16, 128, 4, 'bidirectional').sum()) == 71680


def test_shard_plan():
    assert shard.plan(8, 16, 1) == [shard.Shard(0, 8, 0, 16)]
    assert [tuple(s) for s in shard.plan(8, 16, 4)] == [(0, 2, 0, 16), (2, 4, 0, 16), (4, 6, 0, 16), (6, 8, 0, 16)]
    p = shard.plan(2, 16, 8)
    assert len(p) == 8 and tuple(p[0]) == (0, 1, 0, 4) and tuple(p[7]) == (1, 2, 12, 16)
    with pytest.raises(ValueError):
        shard.plan(3, 16, 2)
    lay = tbs.layouts.fixed(4, 8, 4, 'unidirectional')
    per = int(lay[0].sum())
    assert shard.block_range(lay, 1, 3) == (per, 3 * per)


def test_bind_near_gpu_with_a_fake_nvml(monkeypatch):
    """host.bind_near_gpu: sysfs hidden (as in a container), the CPU set comes from NVML; the
    process is restricted to the cores that are both next to the GPU and available to it, and
    nothing changes when there are none.  NVML and the device query are fakes: no GPU needed."""
    import os
    import sys
    import types
    import torch
    from torch_blocksparse_b200 import host

    avail = sorted(os.sched_getaffinity(0))
    near = set(avail[: max(1, len(avail) // 2)])
    calls = {}

    class Props:
        pci_domain_id, pci_bus_id, pci_device_id = 0, 0x1b, 0
    fake = types.ModuleType('pynvml')
    fake.NVMLError = Exception
    fake.nvmlInit = lambda: calls.setdefault('init', True)
    fake.nvmlShutdown = lambda: calls.setdefault('shutdown', True)

    def by_bus(bus):
        calls['bus'] = bus
        return 'handle'
    fake.nvmlDeviceGetHandleByPciBusId = by_bus

    def affinity(handle, words):
        mask = [0] * words
        for c in calls['cpus']:
            mask[c // 64] |= 1 << (c % 64)
        return mask
    fake.nvmlDeviceGetCpuAffinity = affinity
    fake.nvmlDeviceGetNumaNodeId = lambda handle: 1
    monkeypatch.setitem(sys.modules, 'pynvml', fake)
    monkeypatch.setattr(torch.cuda, 'get_device_properties', lambda device: Props())
    real_open = open

    def no_sysfs(path, *a, **k):
        if str(path).startswith('/sys/bus/pci'):
            raise OSError('hidden')
        return real_open(path, *a, **k)
    monkeypatch.setattr('builtins.open', no_sysfs)
    before = os.sched_getaffinity(0)
    try:
        calls['cpus'] = near
        assert host.bind_near_gpu('cuda:0') == 1
        assert os.sched_getaffinity(0) == near
        assert calls['bus'] == b'00000000:1b:00.0' and calls.get('shutdown')
        os.sched_setaffinity(0, before)
        calls['cpus'] = {max(avail) + 1000}                     # cores this process may not use
        assert host.bind_near_gpu('cuda:0') is None
        assert os.sched_getaffinity(0) == before
    finally:
        os.sched_setaffinity(0, before)
