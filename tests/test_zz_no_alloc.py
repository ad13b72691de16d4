"""pet_gemm_host_static: the weight GEMM for callers that must not allocate device memory.

Some users of this library cannot call cudaMalloc: a plug-in inside a program whose own pool
already holds the whole device, code running while another part of the process has a stream
capture open (cudaMalloc is an error then), a loop that may not wait on the driver's allocator.
For them the library keeps a fixed staging array in its own image and this entry point uses it
instead of the calculator's growable pool.  The test calls it through the C ABI twice in a row (the second call reuses the
array with the first call's contents still in it) and holds it to the allocating entry point's
answer, then checks that an oversized problem is refused with a message.

The file is named so that pytest collects it last.
"""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def fp(a):
    return a.ctypes.data_as(C.POINTER(C.c_float))


def static_gemm(lib, A, W):
    m, k = A.shape
    n = W.shape[0]
    out = np.full((m, n), np.nan, np.float32)
    err = C.create_string_buffer(512)
    rc = lib.pet_gemm_host_static(m, n, k, fp(A), fp(W), fp(out), err, len(err))
    return rc, out, err.value.decode()


def test_static_gemm_matches_the_allocating_entry_point(lib_path, models):
    from pet_kokkos_b200 import Calculator
    from pet_kokkos_b200.calculator import load_library
    lib = load_library()
    calc = Calculator(*models("tiny"))
    rng = np.random.default_rng(7)
    shapes = [(300, 192, 256), (513, 64, 128)]  # (m, n, k); the second, smaller call lands on the first one's leftovers
    for m, n, k in shapes:
        A = rng.normal(size=(m, k)).astype(np.float32)
        W = rng.normal(size=(n, k)).astype(np.float32)
        want = calc.gemm(A, W, "native", w_transposed=True)
        rc, got, msg = static_gemm(lib, A, W)
        assert rc == 0, msg
        # the same kernel on the same numbers: the native GEMM test's band (1e-6 of the largest entry) holds trivially
        assert np.abs(got - want).max() <= 1e-6 * np.abs(want).max()
        ref = A.astype(np.float64) @ W.T.astype(np.float64)
        assert np.abs(got - ref).max() <= 1e-6 * np.abs(ref).max()
    # a repeat of the first problem after the second: nothing stale leaks through
    m, n, k = shapes[0]
    A = rng.normal(size=(m, k)).astype(np.float32)
    W = rng.normal(size=(n, k)).astype(np.float32)
    rc, got, msg = static_gemm(lib, A, W)
    assert rc == 0, msg
    assert np.abs(got - calc.gemm(A, W, "native")).max() <= 1e-6 * np.abs(got).max()
    calc.close()


def test_static_gemm_refuses_what_does_not_fit(lib_path):
    from pet_kokkos_b200.calculator import load_library
    lib = load_library()
    A = np.zeros((4096, 1024), np.float32)
    W = np.zeros((1024, 1024), np.float32)
    rc, _, msg = static_gemm(lib, A, W)
    assert rc == 2 and "exceeds the fixed staging array" in msg
    rc, _, msg = static_gemm(lib, np.zeros((8, 6), np.float32), np.zeros((8, 6), np.float32))
    assert rc == 2 and "multiples of 4" in msg


def test_static_gemm_runs_while_another_stream_is_being_captured(lib_path):
    """One of the callers this entry point is for: while some other part of the process has a stream capture open in
    the global mode, cudaMalloc and anything on the process-wide default stream are errors that also spoil the
    capture. The call does neither (fixed array, the calling thread's own stream), so it must succeed in the middle
    of a capture and the capture must still end and replay cleanly. The device's first call, which looks the array's
    address up, is made before the capture opens, as the header asks."""
    import torch
    from pet_kokkos_b200.calculator import load_library
    lib = load_library()
    rng = np.random.default_rng(11)
    A = rng.normal(size=(200, 64)).astype(np.float32)
    W = rng.normal(size=(96, 64)).astype(np.float32)
    ref = A.astype(np.float64) @ W.T.astype(np.float64)
    rc, got, msg = static_gemm(lib, A, W)
    assert rc == 0, msg
    x = torch.zeros(4096, device="cuda")
    torch.cuda.synchronize()
    side = torch.cuda.Stream()
    graph = torch.cuda.CUDAGraph()
    rc, inside, msg = 1, None, "not called"
    with torch.cuda.graph(graph, stream=side, capture_error_mode="global"):
        y = x + 1.0
        rc, inside, msg = static_gemm(lib, A, W)
        if rc == 0:  # a failed call has spoiled the capture: nothing more goes into it, the assert below reports
            z = y * 2.0
    assert rc == 0, msg
    assert np.abs(inside - ref).max() <= 1e-6 * np.abs(ref).max()
    graph.replay()
    torch.cuda.synchronize()
    assert float(z.sum().item()) == 2.0 * 4096
