"""The allocation-free convolution entry point against the ordinary one and against the CPU oracle.

``mlel_cuda_conv2d_static_scratch`` exists for hosts that cannot call the CUDA allocator where they need
a convolution (a layer's dispatch hook, code inside another runtime's fixed memory budget): it keeps all
of its working memory in an array built into the library.  It must give exactly the bytes that
``mlel_cuda_conv2d`` gives, and both must give the oracle's.  Two calls are made back to back with different
shapes and data, because the built-in array is shared and keeps the previous call's contents: the second
call must not be disturbed by what the first one left behind.  The amount of device memory in use must be
the same after the calls as before them.  Oversized or inconsistent problems must be refused with a message.

This file sorts last on purpose, so that a run that stops at the first failure has already executed
every other test; it also passes when run alone in a fresh process.
"""
import ctypes

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _conv_both_ways(mlel, torch, seed, n, h, w, ic, oc, k, pad, stride, dil, in_zp):
    rng = np.random.Generator(np.random.PCG64(seed))
    x = rng.integers(-128, 128, (n, h, w, ic), dtype=np.int8)
    wt = rng.integers(-128, 128, (oc, k, k, ic), dtype=np.int8)
    b = rng.integers(-(1 << 14), 1 << 14, (oc,), dtype=np.int32)
    oh = (h + 2 * pad - (k - 1) * dil - 1) // stride + 1
    ow = (w + 2 * pad - (k - 1) * dil - 1) // stride + 1
    dx, dw, db = (torch.from_numpy(a).cuda() for a in (x, wt, b))
    out_ref = torch.zeros((n, oh, ow, oc), dtype=torch.int32, device="cuda")
    out_new = torch.full((n, oh, ow, oc), -1, dtype=torch.int32, device="cuda")
    T = mlel.device_tensor
    tx, tw, tb = T(dx.data_ptr(), mlel.I8, x.shape), T(dw.data_ptr(), mlel.I8, wt.shape), T(db.data_ptr(), mlel.I32, b.shape)
    t_ref, t_new = T(out_ref.data_ptr(), mlel.I32, out_ref.shape), T(out_new.data_ptr(), mlel.I32, out_new.shape)
    i32x4 = (ctypes.c_int32 * 4)(pad, pad, pad, pad)
    i32s = (ctypes.c_int32 * 2)(stride, stride)
    i32d = (ctypes.c_int32 * 2)(dil, dil)
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    lib = mlel.lib()
    mlel.check(lib.mlel_cuda_conv2d(ctypes.byref(tx), ctypes.byref(tw), ctypes.byref(tb), ctypes.byref(t_ref), i32x4,
                                    i32s, i32d, in_zp, 0, stream))
    mlel.check(lib.mlel_cuda_conv2d_static_scratch(ctypes.byref(tx), ctypes.byref(tw), ctypes.byref(tb),
                                                   ctypes.byref(t_new), i32x4, i32s, i32d, in_zp, 0, stream))
    torch.cuda.synchronize()
    from oracle import oracle
    want = oracle.conv2d(x, wt, b, [pad] * 4, [stride] * 2, [dil] * 2, in_zp, 0)
    return out_ref.cpu().numpy(), out_new.cpu().numpy(), want


def _device_memory_in_use(torch):
    free, total = torch.cuda.mem_get_info()  # cudaMemGetInfo: what the driver has handed out, whoever asked
    return total - free


def test_static_scratch_conv_matches_the_ordinary_entry_point_twice_in_a_row(mlel):
    import torch
    # first call: an RGB stem (channel count 3, 7x7 stride 2, padding 3, non-zero input zero point)
    ref1, new1, want1 = _conv_both_ways(mlel, torch, 1, n=2, h=37, w=41, ic=3, oc=32, k=7, pad=3, stride=2, dil=1,
                                        in_zp=-3)
    np.testing.assert_array_equal(new1, want1)
    np.testing.assert_array_equal(ref1, want1)
    # second call: smaller problem, other channel count, dilation; reuses the same built-in array
    ref2, new2, want2 = _conv_both_ways(mlel, torch, 2, n=1, h=19, w=17, ic=20, oc=48, k=3, pad=2, stride=1, dil=2,
                                        in_zp=11)
    np.testing.assert_array_equal(new2, want2)
    np.testing.assert_array_equal(ref2, want2)
    assert mlel.lib().mlel_device_error() == 0


def test_static_scratch_conv_leaves_device_memory_as_it_found_it(mlel):
    """The call makes no device allocation: with all operands allocated beforehand (and the first call on the
    device, which resolves the built-in array's address, already made), the driver's count of memory in use is the
    same before and after two more calls."""
    import torch
    rng = np.random.Generator(np.random.PCG64(5))
    n, h, w, ic, oc, k = 2, 24, 24, 16, 32, 3
    x = torch.from_numpy(rng.integers(-128, 128, (n, h, w, ic), dtype=np.int8)).cuda()
    wt = torch.from_numpy(rng.integers(-128, 128, (oc, k, k, ic), dtype=np.int8)).cuda()
    b = torch.from_numpy(rng.integers(-100, 100, (oc,), dtype=np.int32)).cuda()
    out = torch.zeros((n, h, w, oc), dtype=torch.int32, device="cuda")
    T = mlel.device_tensor
    args = (ctypes.byref(T(x.data_ptr(), mlel.I8, x.shape)), ctypes.byref(T(wt.data_ptr(), mlel.I8, wt.shape)),
            ctypes.byref(T(b.data_ptr(), mlel.I32, b.shape)), ctypes.byref(T(out.data_ptr(), mlel.I32, out.shape)),
            (ctypes.c_int32 * 4)(1, 1, 1, 1), (ctypes.c_int32 * 2)(1, 1), (ctypes.c_int32 * 2)(1, 1), 4, 0,
            ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    lib = mlel.lib()
    mlel.check(lib.mlel_cuda_conv2d_static_scratch(*args))  # first call on the device: set-up
    torch.cuda.synchronize()
    before = _device_memory_in_use(torch)
    for _ in range(2):
        mlel.check(lib.mlel_cuda_conv2d_static_scratch(*args))
    torch.cuda.synchronize()
    assert _device_memory_in_use(torch) == before
    from oracle import oracle
    want = oracle.conv2d(x.cpu().numpy(), wt.cpu().numpy(), b.cpu().numpy(), [1] * 4, [1, 1], [1, 1], 4, 0)
    np.testing.assert_array_equal(out.cpu().numpy(), want)


def test_static_scratch_conv_refuses_what_does_not_fit(mlel):
    import torch
    # 64 x 112 x 112 pixels x 160 bytes is far beyond the 32 MiB built-in array
    n, h, w, ic, oc, k = 64, 224, 224, 3, 64, 7
    x = torch.zeros((1,), dtype=torch.int8, device="cuda")  # never dereferenced: the call must fail before launching
    T = mlel.device_tensor
    tx, tw = T(x.data_ptr(), mlel.I8, (n, h, w, ic)), T(x.data_ptr(), mlel.I8, (oc, k, k, ic))
    tb, to = T(x.data_ptr(), mlel.I32, (oc,)), T(x.data_ptr(), mlel.I32, (n, 112, 112, oc))
    pad, st, dl = (ctypes.c_int32 * 4)(3, 3, 3, 3), (ctypes.c_int32 * 2)(2, 2), (ctypes.c_int32 * 2)(1, 1)
    with pytest.raises(mlel.MlelError) as e:
        mlel.check(mlel.lib().mlel_cuda_conv2d_static_scratch(ctypes.byref(tx), ctypes.byref(tw), ctypes.byref(tb),
                                                              ctypes.byref(to), pad, st, dl, 0, 0, None))
    assert "working memory" in str(e.value)


def test_static_scratch_conv_refuses_inconsistent_arguments(mlel):
    import torch
    x = torch.zeros((1,), dtype=torch.int8, device="cuda")  # never dereferenced
    T = mlel.device_tensor
    tx, tw = T(x.data_ptr(), mlel.I8, (1, 8, 8, 16)), T(x.data_ptr(), mlel.I8, (16, 3, 3, 16))
    tb = T(x.data_ptr(), mlel.I32, (16,))
    pad, st, dl = (ctypes.c_int32 * 4)(1, 1, 1, 1), (ctypes.c_int32 * 2)(1, 1), (ctypes.c_int32 * 2)(1, 1)
    lib = mlel.lib()
    good = T(x.data_ptr(), mlel.I32, (1, 8, 8, 16))
    with pytest.raises(mlel.MlelError) as e:  # a zero point that an int8 copy of the input cannot hold
        mlel.check(lib.mlel_cuda_conv2d_static_scratch(ctypes.byref(tx), ctypes.byref(tw), ctypes.byref(tb),
                                                       ctypes.byref(good), pad, st, dl, 200, 0, None))
    assert "zero point" in str(e.value)
    wrong = T(x.data_ptr(), mlel.I32, (1, 7, 8, 16))
    with pytest.raises(mlel.MlelError) as e:  # output height that does not follow from the geometry
        mlel.check(lib.mlel_cuda_conv2d_static_scratch(ctypes.byref(tx), ctypes.byref(tw), ctypes.byref(tb),
                                                       ctypes.byref(wrong), pad, st, dl, 0, 0, None))
    assert "output size" in str(e.value)
