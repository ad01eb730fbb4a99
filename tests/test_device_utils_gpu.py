"""mp* device utilities through the C ABI: stream-ordered memory, copies through
pinned host memory, events ordering two streams, status word, wrapped streams."""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def test_alloc_copy_roundtrip_and_events(mp, stream):
    import torch
    lib = mp.lib()
    n = 1 << 20
    nbytes = n * 4
    h_in = lib.mpHostAlloc(nbytes); h_out = lib.mpHostAlloc(nbytes)
    src = np.ctypeslib.as_array(C.cast(h_in, C.POINTER(C.c_float)), shape=(n,))
    dst = np.ctypeslib.as_array(C.cast(h_out, C.POINTER(C.c_float)), shape=(n,))
    src[:] = np.arange(n, dtype=np.float32); dst[:] = 0
    d_a = lib.mpMemAlloc(nbytes, stream.ctx); d_b = lib.mpMemAlloc(nbytes, stream.ctx)
    assert d_a and d_b
    other = mp.Stream()
    ev = lib.mpEventCreate()
    lib.mpMemcpyHtoD(d_a, h_in, nbytes, stream.ctx)
    lib.launch_dilate_r32(d_a, 2.0, d_b, n, stream.ctx)          # b = 2a on the first stream
    lib.mpEventRecord(ev, stream.ctx)
    lib.mpStreamWaitEvent(other.ctx, ev)                          # second stream waits for it
    lib.launch_translate_r32(d_b, 1.0, d_b, n, other.ctx)         # b = b + 1
    lib.mpMemcpyDtoH(h_out, d_b, nbytes, other.ctx)
    other.sync()
    assert np.array_equal(dst, 2 * np.arange(n, dtype=np.float32) + 1)
    lib.mpMemFree(d_a, stream.ctx); lib.mpMemFree(d_b, stream.ctx)
    stream.sync()
    lib.mpEventDestroy(ev); other.close()
    lib.mpHostFree(h_in); lib.mpHostFree(h_out)
    assert stream.status() == 0
    assert lib.mpWorkspaceBytes(stream.ctx) >= 1 << 20
    assert lib.mpDeviceSmCount(stream.ctx) == torch.cuda.get_device_properties(0).multi_processor_count
    assert lib.mpDeviceTotalMemory(0) == torch.cuda.get_device_properties(0).total_memory


def test_wrapped_torch_stream(mp):
    import torch
    s = mp.Stream(wrap=torch.cuda.current_stream().cuda_stream)
    x = torch.randn(1000, device="cuda"); y = torch.empty_like(x)
    mp.launch("relu", torch.float32, x, y, 1000, s)              # ordered on torch's own stream
    assert torch.equal(y, torch.relu(x))
    s.close()
    assert float(x.sum()) == float(x.sum())                       # torch's stream is still alive
