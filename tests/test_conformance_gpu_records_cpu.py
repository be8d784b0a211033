"""Record and handle types of ``ferrotorch_b200.gpu`` that need no device: allocator / guard statistics, reservations, pool handles, the
error base, and the argument checks of device-only entry points when given host tensors."""
import pytest
import torch

from ferrotorch_b200 import errors
from ferrotorch_b200 import gpu as G


def test_statistics_records_and_reservations():
    s = G.AllocatorStats(10, 20, 15, 25, 3, 1, 2, 1, 0, 2)
    assert (s.allocated, s.reserved, s.peak_allocated, s.num_allocs, s.live_blocks) == (10, 20, 15, 3, 2)
    g = G.MemoryGuard(1000, query=lambda: (100, 2000))
    r = g.reserve(300)
    assert isinstance(r, G.MemoryReservation)
    st = g.stats()
    assert isinstance(st, G.MemoryGuardStats) and st.budget == 1000 and st.reserved_by_guard == 300 and st.used == 400 and st.oom_events == 0
    r.release()
    r.release()                                   # idempotent
    assert g.stats().reserved_by_guard == 0
    h = G.GraphPoolHandle(7)
    assert h.id == 7 and h == G.GraphPoolHandle(7)
    assert issubclass(G.GpuError, errors.FerrotorchError) and issubclass(G.OutOfMemory, Exception)
    assert [p.name for p in G.StreamPriority] == ["HIGH", "NORMAL"] and int(G.StreamPriority.HIGH) == -1


def test_device_entry_points_refuse_host_tensors():
    a, b, out = torch.ones(4), torch.ones(4), torch.empty(4)
    for call in (lambda: G.gpu_mul_into(a, b, out), lambda: G.gpu_gelu(a), lambda: G.gpu_mul_bf16(a.bfloat16(), b.bfloat16()),
                 lambda: G.gpu_small_matmul_into(a, b, out, 2, 2, 2), lambda: G.gpu_bmm_f32_into(a, b, out, 1, 2, 2, 2)):
        with pytest.raises(Exception) as ei:
            call()
        assert "cuda" in str(ei.value).lower() or "device" in str(ei.value).lower() or isinstance(ei.value, errors.FerrotorchError)
    assert G.tensor_to_cpu(a) is a
    assert callable(G.install_as_torch_allocator) and callable(G.torch_allocator) and callable(G.begin_capture_with_pool) and callable(G.GraphCaptureGuard)
    assert G.CudaBackendImpl is not None and callable(G.cpu_to_gpu_pinned) and callable(G.alloc_zeros_f64)
