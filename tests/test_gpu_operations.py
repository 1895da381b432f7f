"""Owned asynchronous operations and the bounded host wait through the C ABI
(crates/fe2o3-core/src/operation.rs:272-420, crates/fe2o3-core/src/memory.rs:129-161,
crates/fe2o3-completion/src/lib.rs:46-60).  Nothing here faults or hangs a GPU: the
"ambiguous" outcomes are produced by a host deadline of zero milliseconds on work
that simply has not finished yet.
"""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def gpu():
    import fe2o3_b200 as fe
    ctx = fe.GpuContext(0)
    return fe, ctx, ctx.create_stream()


def _reduce_setup(fe, ctx, stream, n):
    from fe2o3_b200 import synth
    hv, ha, ho = ctx.pinned(n, np.uint32), ctx.pinned(n, np.uint32), ctx.pinned(1, np.uint32)
    synth.u32_below(1, 1, n, 1 << 16, out=hv)
    synth.bernoulli(1, 2, n, 0.75, flag_value=7, packed=False, flags_out=ha)
    v, a = fe.DeviceBuffer.zeroed(stream, n, np.uint32), fe.DeviceBuffer.zeroed(stream, n, np.uint32)
    o = fe.DeviceBuffer.zeroed(stream, 1, np.uint32)
    prep = fe.prepare(ctx, "masked_reduce_u32", values=v, active=a, output=o)
    return hv, ha, ho, v, a, o, prep


def test_operation_owns_its_buffers_until_completion(gpu, orc):
    fe, ctx, stream = gpu
    n = 1 << 26
    hv, ha, ho, v, a, o, prep = _reduce_setup(fe, ctx, stream, n)
    ho[0] = 0xdeadbeef
    op = fe.Operation.submit(stream, prep, buffers=(), copies_in=[(v, hv), (a, ha)], copies_out=[(o, ho)])
    # 512 MiB over PCIe are still on their way: the buffers cannot be freed now
    for buf in (v, a, o):
        with pytest.raises(fe.Fe2o3Error) as err:
            buf.free()
        assert err.value.status == -17      # Busy: owned by a submitted operation
    assert op.wait(20000) == 0
    assert int(ho[0]) == orc.masked_sum_u32(hv, ha)
    for buf in (v, a, o):
        buf.free()                          # released at completion


def test_wait_deadline_leaves_the_operation_submitted(gpu, orc):
    fe, ctx, stream = gpu
    n = 1 << 26
    hv, ha, ho, v, a, o, prep = _reduce_setup(fe, ctx, stream, n)
    op = fe.Operation.submit(stream, prep, copies_in=[(v, hv), (a, ha)], copies_out=[(o, ho)])
    with pytest.raises(fe.Fe2o3Error) as err:
        op.wait(0)                          # a zero deadline on work that takes milliseconds
    assert err.value.status == -18          # StillRunning: the operation stays submitted
    with pytest.raises(fe.Fe2o3Error):
        v.free()                            # still owned
    assert op.wait(20000) == 0              # the same operation can be waited for again
    assert int(ho[0]) == orc.masked_sum_u32(hv, ha)
    for buf in (v, a, o):
        buf.free()


def test_abandoned_operation_quarantines_its_buffers(gpu):
    fe, ctx, stream = gpu
    n = 1 << 20
    hv, ha, ho, v, a, o, prep = _reduce_setup(fe, ctx, stream, n)
    op = fe.Operation.submit(stream, prep, copies_in=[(v, hv), (a, ha)], copies_out=[(o, ho)])
    op.abandon()                            # completion was never established
    for buf in (v, a, o):
        buf.free()                          # accepted, and deliberately leaks the device memory (memory.rs:129-161)
    stream.synchronize()                    # the work itself finishes normally; nothing was freed under it


def test_dispatch_and_wait_deadline_is_ambiguous_not_fatal(gpu, orc):
    """launch_and_wait with a zero host deadline on a 2^28-element reduction: AmbiguousCompletion, nothing
    freed, the stream still usable, and the result correct once the stream has been synchronised."""
    fe, ctx, stream = gpu
    n = 1 << 28
    hv, ha, ho, v, a, o, prep = _reduce_setup(fe, ctx, stream, n)
    v.copy_from_host_async(stream, hv)
    a.copy_from_host_async(stream, ha)
    stream.synchronize()
    with pytest.raises(fe.Fe2o3Error) as err:
        prep.launch_and_wait(stream, 0)
    assert err.value.status == -11 and "AmbiguousCompletion" in str(err.value)
    for buf in (v, a, o):
        buf.quarantine()                    # what a caller does with buffers of unknown completion
    stream.synchronize()                    # quiescence can still be established later
    assert ctx.take_kernel_status(stream) == 0
    o.copy_to_host_async(stream, ho)
    stream.synchronize()
    assert int(ho[0]) == orc.masked_sum_u32(hv, ha)
    for buf in (v, a, o):
        buf.free()                          # a quarantined buffer's free is a leak by design, and succeeds
