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


def test_graph_capture_replays_a_launch_sequence(mp):
    """mpGraphBeginCapture / EndCapture / Launch: three dependent launches recorded once reproduce the eagerly
    computed result on every replay, also after the inputs change in place."""
    import numpy as np
    import torch
    lib = mp.lib()
    s = mp.Stream()
    n = 1 << 16
    a = torch.randn(n, device="cuda"); b = torch.randn(n, device="cuda")
    t = torch.empty_like(a); out = torch.empty_like(a)
    torch.cuda.synchronize()

    def chain():
        mp.launch("addition", torch.float32, a, b, t, n, s)
        mp.launch("selu", torch.float32, t, out, n, s)
        mp.launch("hadamard", torch.float32, out, a, out, n, s)

    chain(); s.sync()
    want = out.clone()
    lib.mpGraphBeginCapture(s.ctx)
    chain()
    g = lib.mpGraphEndCapture(s.ctx)
    assert g
    out.zero_(); torch.cuda.synchronize()
    lib.mpGraphLaunch(g, s.ctx); s.sync()
    assert torch.equal(out, want)
    a.mul_(2.0); torch.cuda.synchronize()          # same buffers, new contents
    lib.mpGraphLaunch(g, s.ctx); s.sync()
    ref = torch.nn.functional.selu(a + b) * a
    assert float((out - ref).abs().max()) < 1e-5
    assert s.status() == 0
    lib.mpGraphDestroy(g)
    s.close()


def test_ssd_helper_streams_are_released(mp):
    """A stream that ran the scan (which forks helper streams) can be closed and re-created."""
    import torch
    for _ in range(2):
        s = mp.Stream()
        dims = (1, 256, 2, 64, 128, 1, 128)
        x = torch.randn(1, 256, 2, 64, device="cuda").half(); Bm = torch.randn(1, 256, 1, 128, device="cuda").half()
        Cm = torch.randn(1, 256, 1, 128, device="cuda").half(); dt = torch.rand(1, 256, 2, device="cuda") * 0.1
        A = -torch.ones(2, device="cuda"); y = torch.empty_like(x)
        scr = torch.empty(mp.lib().mpSsdScanScratchBytes(*dims, 0), dtype=torch.uint8, device="cuda")
        torch.cuda.synchronize()
        mp.launch("ssd_scan", torch.float16, x, dt, A, Bm, Cm, y, scr, *dims, s)
        s.sync()
        assert s.status() == 0 and bool(torch.isfinite(y).all())
        s.close()


def test_a_wait_that_cannot_be_satisfied_times_out_and_reports(mp):
    """The bounded waits' time-out path, exercised without a fault: with a 1 ms limit a kernel that waits for a
    barrier phase nobody completes returns by itself, the status word reads MP_STATUS_WAIT_TIMEOUT, and the stream
    stays usable."""
    import time
    import torch
    torch.zeros(1, device="cuda")
    lib = mp.lib()
    with mp.Stream() as s:
        lib.mpSetWaitLimit(s.ctx, 1000)
        t0 = time.monotonic()
        lib.mpSelfTestWaitTimeout(s.ctx)
        s.sync()
        assert time.monotonic() - t0 < 1.0           # far below the default 2 s: the run-time limit was used
        assert s.status() == 1                       # MP_STATUS_WAIT_TIMEOUT
        assert s.status() == 0                       # reading clears it
        lib.mpSetWaitLimit(s.ctx, 0)
        x = torch.arange(1024, dtype=torch.float32, device="cuda"); y = torch.empty_like(x)
        torch.cuda.synchronize()
        mp.launch("copy", torch.float32, x, y, 1024, s)
        s.sync()
        assert torch.equal(x, y) and s.status() == 0
