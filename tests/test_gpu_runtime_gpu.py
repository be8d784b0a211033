"""Device runtime on a GPU: native allocator over cudaMalloc, streams / events, graph capture helpers, module cache (NVRTC -> native loader), GpuTensor."""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def test_allocator_streams_graphs_modules_and_gputensor():
    from ferrotorch_b200 import _lib, gpu
    be = gpu.init_cuda_backend(0)
    assert be.abi >= 1 and be.device.sm_count >= 100 and gpu.gpu_backend() is be
    a = gpu.CudaAllocator()
    p1, p2 = a.malloc(1 << 20), a.malloc(3 << 20)
    assert p1 and p2 and a.stats().reserved >= 4 << 20
    # the memory is usable: wrap it and run a kernel on it
    n = (1 << 20) // 4
    arr = (ctypes.c_float * 4).from_buffer_copy(bytes(16))
    _lib.call("ft_ew_fill", 0, p1, n, 2.5, _lib.S())
    out = torch.empty(n, device="cuda")
    _lib.call("ft_ew_unary", 0, 24, p1, out, n, 2.0, 1.0, _lib.S())        # scale: x * 2 + 1
    assert float(out.sum()) == 6.0 * n
    a.free(p1)
    assert a.malloc(1 << 20) == p1                                           # cached block re-used
    a.free(p2)
    a.free(p1)
    assert a.empty_cache() >= 4 << 20 and a.stats().reserved == 0
    a.close()
    pool = gpu.StreamPool(size=4)
    s = pool.next()
    e0, e1 = gpu.CudaEventWrapper(), gpu.CudaEventWrapper()
    with gpu.StreamGuard(s):
        e0.record()
        x = torch.randn(1024, 1024, device="cuda")
        y = x @ x
        e1.record()
    e1.synchronize()
    assert e0.elapsed_ms(e1) > 0 and e1.query() and pool.next() is not s
    pos = gpu.DeviceScalar(3)
    buf = torch.zeros(8, device="cuda")

    def body(t):
        return t * 2 + pos.tensor().float()
    g = gpu.make_graphed_callable(body, (torch.ones(8, device="cuda"),))
    assert torch.equal(g(torch.full((8,), 2.0, device="cuda")), torch.full((8,), 7.0, device="cuda"))
    pos.set(10)
    assert torch.equal(g(torch.ones(8, device="cuda")), torch.full((8,), 12.0, device="cuda")) and g.graph.launches >= 0
    mc = gpu.ModuleCache()
    src = 'extern "C" __global__ void axpy(float a, const float* x, float* y, int n) { int i = blockIdx.x * blockDim.x + threadIdx.x; if (i < n) y[i] += a * x[i]; }'
    k = mc.get_or_compile("axpy", src)
    assert mc.get_or_compile("axpy", src) == k and mc.compiles == 1 and mc.hits == 1
    xs, ys = torch.arange(1000.0, device="cuda"), torch.ones(1000, device="cuda")
    mc.launch(k, 4, 256, [ctypes.c_float(0.5), ctypes.c_void_p(xs.data_ptr()), ctypes.c_void_p(ys.data_ptr()), ctypes.c_int(1000)])
    assert torch.allclose(ys, 1 + 0.5 * torch.arange(1000.0, device="cuda"))
    t = gpu.GpuTensor.from_host([1.0, -2.0, 3.0, -4.0], (2, 2))
    assert t.add(t).neg().relu().to_host().tolist() == [[0.0, 4.0], [0.0, 8.0]] and t.try_clone().cu_device_ptr() != t.cu_device_ptr()
    mgr = gpu.CudaRngManager(seed=5)
    mgr.fork_rng()
    a1 = mgr.generator(0).uniform_(torch.empty(100, device="cuda"))
    mgr.join_rng()
    assert torch.equal(a1, mgr.generator(0).uniform_(torch.empty(100, device="cuda")))
    guard = gpu.MemoryGuard()
    with guard.reserve(1 << 20):
        assert guard.stats().reserved_by_guard == 1 << 20
    assert _lib.read_status() == 0
