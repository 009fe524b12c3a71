"""Data pipeline, profiling / fusion / layout / sparse utilities and the CPU-visible part of the device API."""
import pytest
import torch

from ghost_flow_b200 import cuda as gf_cuda
from ghost_flow_b200 import data as D
from ghost_flow_b200 import utils as U


def test_datasets_samplers_loader():
    x, y = torch.arange(40.0).view(20, 2), torch.arange(20)
    ds = D.TensorDataset(x, y)
    assert len(ds) == 20 and torch.equal(ds[3][0], x[3])
    assert len(D.ConcatDataset([ds, D.Subset(ds, [0, 1, 2])])) == 23
    dl = D.DataLoader(ds, batch_size=6, shuffle=True, seed=1)
    seen = torch.cat([b[1] for b in dl])
    assert sorted(seen.tolist()) == list(range(20)) and len(dl) == 4
    assert len(D.DataLoader(ds, batch_size=6).drop_last()) == 3
    # rank-contiguous shards that together cover everything exactly once
    parts = [list(D.DistributedSampler(20, 3, r)) for r in range(3)]
    assert sorted(sum(parts, [])) == list(range(20))
    tok = D.SyntheticTokenDataset(100, 16, 8, seed=0)
    a, b = tok[0]
    assert a.shape == (16,) and torch.equal(a[1:], b[:-1]) and int(a.max()) < 100
    w = D.WeightedRandomSampler([0.0, 0.0, 1.0], 10)
    assert set(w) == {2}


def test_transforms():
    img = torch.rand(3, 8, 8)
    t = D.Compose([D.Normalize([0.5] * 3, [0.5] * 3), D.RandomHorizontalFlip(1.0), D.RandomCrop(6, padding=1)])
    out = t(img)
    assert out.shape == (3, 6, 6)
    assert torch.allclose(D.RandomHorizontalFlip(1.0)(img), img.flip(-1))
    assert D.RandomErasing(1.0, value=0.0)(img).eq(0).any()


def test_profiler_benchmark_memory_pool():
    prof = U.Profiler(use_cuda_events=False)
    with prof.start("step"):
        torch.randn(64, 64) @ torch.randn(64, 64)
    with prof.start("step"):
        pass
    s = prof.summary()
    assert s["step"]["count"] == 2 and s["step"]["total_ms"] >= 0
    r = U.Benchmark("mm").warmup(1).iterations(3).run(lambda: torch.randn(32, 32) @ torch.randn(32, 32))
    assert r.iterations == 3 and r.mean > 0 and r.min <= r.median <= r.max
    pool = U.MemoryPool()
    a = pool.allocate(1000)
    pool.deallocate(a)
    b = pool.allocate(900)
    st = pool.get_stats()
    assert st.reuse_rate() > 0 and b.data_ptr() == a.data_ptr()


def test_fusion_layout_hardware_sparse():
    eng = U.FusionEngine()
    found = eng.analyze(["Conv2d", "BatchNorm2d", "ReLU", "Linear", "ReLU", "Tanh"])
    assert found == [(0, U.FusionPattern.ConvBNReLU), (3, U.FusionPattern.LinearReLU)]
    assert eng.kernel_for(U.FusionPattern.ConvBNReLU) == "gf_conv_bn_relu" and eng.estimate_speedup(U.FusionPattern.ConvBNReLU) > 1
    lo = U.LayoutOptimizer()
    x = torch.randn(2, 3, 4, 5)
    assert torch.equal(lo.nhwc_to_nchw(lo.nchw_to_nhwc(x)), x)
    assert any(d.backend is U.HardwareBackend.CPU for d in U.list_devices())
    dense = torch.tensor([[0.0, 2.0, 0.0], [1.0, 0.0, 3.0]])
    coo = U.SparseTensorCOO.from_dense(dense)
    assert coo.nnz() == 3 and torch.equal(coo.to_dense(), dense)
    v = torch.tensor([1.0, 2.0, 3.0])
    assert torch.allclose(coo.spmv(v), dense @ v) and torch.allclose(coo.to_csr().spmv(v), dense @ v)
    assert torch.equal(coo.transpose().to_dense(), dense.t())


def test_device_api_without_a_gpu_reports_cleanly():
    if torch.cuda.is_available():
        pytest.skip("covers the no-GPU behaviour")
    assert gf_cuda.is_available() is False and gf_cuda.device_count() == 0
    with pytest.raises(gf_cuda.CudaError) as e:
        gf_cuda.CudaDevice(0)
    assert e.value.kind is gf_cuda.CudaError.Kind.NotAvailable
    cfg = gf_cuda.LaunchConfig.for_elements(1000, 256)
    assert cfg.grid == (4, 1, 1) and cfg.block == (256, 1, 1)
    assert gf_cuda.GpuMemoryPool.size_class(1000) == 1024 and len(gf_cuda.KERNELS) == 17
