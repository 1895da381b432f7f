"""The allocation-free masked sum against the prepared entry point.

fe2o3_masked_reduce_u32_noalloc serves hosts that cannot call the device
allocator while running (device memory fully owned by another runtime's pool,
or no room for an allocation's device-wide synchronisation); its scratch is a
fixed device array inside the library.  This file is collected last so that a
run stopping at the first failure has already run every other test; it also
passes alone in a fresh process (it makes its own context and buffers).
"""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def test_noalloc_masked_sum_matches_prepared_entry_point_twice(orc):
    import fe2o3_b200 as fe
    from fe2o3_b200 import synth
    from fe2o3_b200._lib import lib

    ctx = fe.GpuContext(0)
    stream = ctx.default_stream()
    fn = lib.fe2o3_masked_reduce_u32_noalloc
    fn.restype = C.c_int32
    fn.argtypes = [C.c_void_p, C.c_void_p, C.c_uint64, C.c_void_p, C.c_void_p]

    for call, n in enumerate([(1 << 22) + 13, 70001, 0]):  # calls in a row share the scratch array
        values = synth.u32_below(11 + call, 1, n, 1 << 16) if n else np.zeros(0, np.uint32)
        if n:
            values[::5] = 0xFFFFFF00  # force wrap-around
        flags = synth.bernoulli(11 + call, 2, n, 0.75, packed=False)[0] if n else np.zeros(0, np.uint32)
        v, a = fe.DeviceBuffer.from_host(stream, values), fe.DeviceBuffer.from_host(stream, flags)
        ref_out = fe.DeviceBuffer.from_host(stream, np.full(1, 0xDEADBEEF, np.uint32))
        new_out = fe.DeviceBuffer.from_host(stream, np.full(1, 0xDEADBEEF, np.uint32))
        fe.prepare(ctx, "masked_reduce_u32", values=v, active=a, output=ref_out).launch_and_wait(stream)
        st = fn(v.as_device_ptr() or None, a.as_device_ptr() or None, n, new_out.as_device_ptr(), stream.native or None)
        assert st == 0, lib.fe2o3_last_error()
        stream.synchronize()
        want = int(ref_out.to_host_vec(stream)[0])
        got = int(new_out.to_host_vec(stream)[0])
        assert got == want == orc.masked_sum_u32(values, flags), (call, got, want)  # integers: bit-exact

    # the same on a stream of the caller's own (not the default stream): the call is asynchronous on it
    own = ctx.create_stream()
    n = 300007
    values, flags = synth.u32_below(21, 1, n, 1 << 16), synth.bernoulli(21, 2, n, 0.75, packed=False)[0]
    v, a = fe.DeviceBuffer.from_host(own, values), fe.DeviceBuffer.from_host(own, flags)
    out = fe.DeviceBuffer.from_host(own, np.full(1, 0xDEADBEEF, np.uint32))
    assert fn(v.as_device_ptr(), a.as_device_ptr(), n, out.as_device_ptr(), own.native) == 0, lib.fe2o3_last_error()
    own.synchronize()
    assert int(out.to_host_vec(own)[0]) == orc.masked_sum_u32(values, flags)

    # sizes beyond the stated maximum are rejected before anything is launched
    one = fe.DeviceBuffer.zeroed(stream, 4, np.uint32)
    st = fn(one.as_device_ptr(), one.as_device_ptr(), (1 << 31) + 1, one.as_device_ptr(), None)
    assert st == -10 and b"allocation-free limit" in lib.fe2o3_last_error()
    assert fn(None, one.as_device_ptr(), 4, one.as_device_ptr(), None) == -7
    assert fn(one.as_device_ptr(), one.as_device_ptr(), 4, None, None) == -7
