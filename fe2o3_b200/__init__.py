"""fe2o3_b200: B200-native kernels behind fe2o3's host surface.

Python mirror of fe2o3-core's `GpuContext / Stream / DeviceBuffer / Event`
(crates/fe2o3-core/src/lib.rs:18-53) and of the generated per-kernel host
adapters' `prepare -> launch` (crates/fe2o3-host/src/generated_vecadd.rs:54-147),
all implemented by calls into the C ABI of libfe2o3_b200.so.
"""
import ctypes as C

import numpy as np

from . import _lib
from ._lib import Fe2o3Error, Slice, check, lib

DROP_ROUTE = 0xFFFFFFFF
SCHEDULE_EXACT_ORDER, SCHEDULE_TCGEN05, SCHEDULE_AUTO = 0, 1, 2
DTYPE_F32, DTYPE_BF16 = 0, 1
ERR_NO_DISPATCH = 1000


class GpuContext:
    """crates/fe2o3-core/src/context.rs:11-62"""

    def __init__(self, device=0):
        self._h = C.c_void_p()
        check(lib.fe2o3_ctx_create(C.c_int32(device), C.byref(self._h)), "GpuContext::new")
        self.device = device

    def default_stream(self):
        h = C.c_void_p()
        check(lib.fe2o3_stream_default(self._h, C.byref(h)), "default_stream")
        return Stream(self, h)

    def create_stream(self):
        h = C.c_void_p()
        check(lib.fe2o3_stream_create(self._h, C.byref(h)), "create_stream")
        return Stream(self, h)

    def wrap_stream(self, cuda_stream):
        h = C.c_void_p()
        check(lib.fe2o3_stream_wrap(self._h, C.c_void_p(cuda_stream), C.byref(h)), "wrap_stream")
        return Stream(self, h)

    def bind_to_thread(self):
        check(lib.fe2o3_ctx_bind_to_thread(self._h), "bind_to_thread")

    def observe_environment(self):
        p = _lib.DeviceProperties()
        check(lib.fe2o3_ctx_observe_environment(self._h, C.byref(p)), "observe_environment")
        return p

    def pinned(self, shape, dtype):
        """Pinned host array (crates/fe2o3-core/src/pinned_memory.rs)."""
        dtype = np.dtype(dtype)
        n = int(np.prod(shape))
        ptr = C.c_void_p()
        check(lib.fe2o3_pinned_alloc(self._h, C.c_uint64(n * dtype.itemsize), C.byref(ptr)), "pinned_alloc")
        buf = (C.c_uint8 * (n * dtype.itemsize)).from_address(ptr.value)
        arr = np.frombuffer(buf, dtype=dtype, count=n).reshape(shape)
        return arr

    def take_kernel_status(self, stream):
        s = C.c_uint32()
        check(lib.fe2o3_ctx_take_kernel_status(self._h, stream._h, C.byref(s)), "take_kernel_status")
        return s.value


class Stream:
    """crates/fe2o3-core/src/stream.rs"""

    def __init__(self, ctx, handle):
        self.ctx, self._h = ctx, handle

    def synchronize(self):
        check(lib.fe2o3_stream_sync(self._h), "Stream::synchronize")

    def wait_event(self, event):
        """Later work on this stream starts after `event` has completed (device-side ordering)."""
        check(lib.fe2o3_stream_wait_event(self._h, event._h), "Stream::wait_event")

    @property
    def native(self):
        p = C.c_void_p()
        check(lib.fe2o3_stream_native(self._h, C.byref(p)), "stream_native")
        return p.value or 0


class DeviceBuffer:
    """crates/fe2o3-core/src/memory.rs:435-492"""

    def __init__(self, handle, dtype, ctx):
        self._h, self.dtype, self.ctx = handle, np.dtype(dtype), ctx

    @classmethod
    def zeroed(cls, stream, elements, dtype):
        h = C.c_void_p()
        dt = np.dtype(dtype)
        check(lib.fe2o3_buf_alloc_zeroed(stream._h, C.c_uint64(elements), C.c_uint32(dt.itemsize), C.byref(h)),
              "DeviceBuffer::zeroed")
        return cls(h, dt, stream.ctx)

    @classmethod
    def from_host(cls, stream, array):
        a = np.ascontiguousarray(array)
        h = C.c_void_p()
        check(lib.fe2o3_buf_from_host(stream._h, a.ctypes.data_as(C.c_void_p), C.c_uint64(a.size),
                                      C.c_uint32(a.dtype.itemsize), C.byref(h)), "DeviceBuffer::from_host")
        return cls(h, a.dtype, stream.ctx)

    def to_host_vec(self, stream):
        out = np.empty(len(self), self.dtype)
        check(lib.fe2o3_buf_to_host(stream._h, self._h, out.ctypes.data_as(C.c_void_p), C.c_uint64(len(self))),
              "DeviceBuffer::to_host_vec")
        return out

    def copy_from_host_async(self, stream, array):
        check(lib.fe2o3_buf_copy_from_host_async(stream._h, self._h, array.ctypes.data_as(C.c_void_p),
                                                 C.c_uint64(array.size)), "copy_from_host_async")

    def copy_to_host_async(self, stream, array):
        check(lib.fe2o3_buf_copy_to_host_async(stream._h, self._h, array.ctypes.data_as(C.c_void_p),
                                               C.c_uint64(array.size)), "copy_to_host_async")

    def __len__(self):
        return int(lib.fe2o3_buf_len(self._h))

    @property
    def __cuda_array_interface__(self):
        """Zero-copy view for array libraries (`torch.as_tensor(buf, device="cuda")`)."""
        return {"shape": (len(self),), "typestr": self.dtype.str, "data": (self.as_device_ptr(), False), "version": 2}

    def as_device_ptr(self):
        return int(lib.fe2o3_buf_ptr(self._h))

    def view(self, start=0, length=None):
        s = Slice()
        length = len(self) - start if length is None else length
        check(lib.fe2o3_buf_slice(self._h, C.c_uint64(start), C.c_uint64(length), C.byref(s)), "DeviceBuffer::view")
        return s

    def quarantine(self):
        check(lib.fe2o3_buf_quarantine(self._h), "quarantine")

    def free(self):
        if self._h:
            check(lib.fe2o3_buf_free(self._h), "DeviceBuffer::drop")
            self._h = None


class Event:
    """crates/fe2o3-core/src/event.rs:82-148"""

    def __init__(self, ctx):
        self._h = C.c_void_p()
        check(lib.fe2o3_event_create(ctx._h, C.byref(self._h)), "Event::new")

    def record(self, stream):
        check(lib.fe2o3_event_record(self._h, stream._h), "Event::record")

    def synchronize(self):
        check(lib.fe2o3_event_sync(self._h), "Event::synchronize")

    def query(self):
        d = C.c_int32()
        check(lib.fe2o3_event_query(self._h, C.byref(d)), "Event::query")
        return bool(d.value)

    def elapsed_time_ms_since(self, start):
        ms = C.c_float()
        check(lib.fe2o3_event_elapsed_ms(start._h, self._h, C.byref(ms)), "Event::elapsed_time_ms_since")
        return ms.value


class Operation:
    """A submitted operation that owns its buffers until completion is established
    (crates/fe2o3-core/src/operation.rs:272-420 OwnedDeviceOperation)."""

    def __init__(self, handle, keep):
        self._h, self._keep = handle, keep   # the host arrays of the copies must outlive the operation

    @classmethod
    def submit(cls, stream, prepared=None, buffers=(), copies_in=(), copies_out=()):
        """copies_in / copies_out: (DeviceBuffer, host array) pairs, host -> device before the launch and
        device -> host after it."""
        def pack(pairs):
            arr = (_lib.HostCopy * max(1, len(pairs)))()
            for i, (buf, host) in enumerate(pairs):
                arr[i].buffer, arr[i].host, arr[i].elements = buf._h, host.ctypes.data, host.size
            return arr
        bufs = (C.c_void_p * max(1, len(buffers)))(*[b._h for b in buffers])
        h = C.c_void_p()
        st = lib.fe2o3_operation_submit(stream._h, prepared._h if prepared else None, bufs, C.c_uint32(len(buffers)),
                                        pack(copies_in), C.c_uint32(len(copies_in)), pack(copies_out),
                                        C.c_uint32(len(copies_out)), C.byref(h))
        op = cls(h, (copies_in, copies_out)) if h.value else None
        if st != 0:
            if op:   # work may be pending: establish quiescence before reporting the submission error
                op.abandon()
            check(st, "Operation::submit")
        return op

    def is_complete(self):
        d = C.c_int32()
        check(lib.fe2o3_operation_is_complete(self._h, C.byref(d)), "Operation::is_complete")
        return bool(d.value)

    def wait(self, timeout_ms=5000):
        """Returns the kernel status word.  A deadline that passes raises Fe2o3Error(StillRunning, -18) and
        leaves the operation submitted; any other outcome consumes it."""
        ks = C.c_uint32()
        st = lib.fe2o3_operation_wait(self._h, C.c_uint32(timeout_ms), C.byref(ks))
        if st == -18:
            check(st, "Operation::wait")
        self._h = None
        check(st, "Operation::wait")
        return ks.value

    def abandon(self):
        if self._h:
            lib.fe2o3_operation_abandon(self._h)
            self._h = None


class PeerRegion:
    """Device memory that the other processes of the node can map
    (crates/fe2o3-core/src/peer_access.rs:24-60 across processes)."""

    HANDLE_BYTES = 64

    def __init__(self, ctx, handle):
        self.ctx, self._h = ctx, handle

    @classmethod
    def create(cls, ctx, nbytes):
        h = C.c_void_p()
        check(lib.fe2o3_peer_region_create(ctx._h, C.c_uint64(nbytes), C.byref(h)), "PeerRegion::create")
        return cls(ctx, h)

    @classmethod
    def open(cls, ctx, handle_bytes):
        h = C.c_void_p()
        buf = (C.c_uint8 * cls.HANDLE_BYTES).from_buffer_copy(bytes(handle_bytes))
        check(lib.fe2o3_peer_region_import(ctx._h, buf, C.byref(h)), "PeerRegion::open")
        return cls(ctx, h)

    def export(self):
        buf = (C.c_uint8 * self.HANDLE_BYTES)()
        check(lib.fe2o3_peer_region_export(self._h, buf), "PeerRegion::export")
        return bytes(buf)

    @property
    def ptr(self):
        return int(lib.fe2o3_peer_region_ptr(self._h))

    @property
    def nbytes(self):
        return int(lib.fe2o3_peer_region_bytes(self._h))

    def close(self):
        if self._h:
            check(lib.fe2o3_peer_region_destroy(self._h), "PeerRegion::close")
            self._h = None


def as_slice(x):
    """DeviceBuffer, Slice, torch tensor, (ptr, len) tuple or None -> Slice."""
    if x is None:
        return Slice(0, 0)
    if isinstance(x, Slice):
        return x
    if isinstance(x, DeviceBuffer):
        return Slice(x.as_device_ptr(), len(x))
    if isinstance(x, tuple):
        return Slice(int(x[0]), int(x[1]))
    if hasattr(x, "data_ptr"):
        return Slice(x.data_ptr() if x.numel() else 0, x.numel())
    raise TypeError(f"cannot make a device slice from {type(x)}")


class Prepared:
    """A checked, packed launch: the generated adapters' `prepare` result."""

    def __init__(self, ctx, handle, op):
        self.ctx, self._h, self.op = ctx, handle, op

    def launch(self, stream):
        check(lib.fe2o3_prepared_launch(self._h, stream._h), f"{self.op}.launch")

    def launch_and_wait(self, stream, timeout_ms=5000):
        ks = C.c_uint32()
        st = lib.fe2o3_prepared_launch_and_wait(self._h, stream._h, C.c_uint32(timeout_ms), C.byref(ks))
        self.kernel_status = ks.value
        check(st, f"{self.op}.dispatch_and_wait")

    @property
    def geometry(self):
        g = _lib.Geometry()
        check(lib.fe2o3_prepared_geometry(self._h, C.byref(g)), "geometry")
        return g

    @property
    def kernarg(self):
        n = C.c_uint64(320)
        buf = (C.c_uint8 * 320)()
        check(lib.fe2o3_prepared_kernarg(self._h, buf, C.byref(n)), "kernarg")
        return bytes(buf[: n.value])

    def patch_kernarg(self, offset, data: bytes):
        """Overwrite scalar bytes of the packed block (e.g. the exchange epoch)."""
        buf = (C.c_uint8 * len(data)).from_buffer_copy(data)
        check(lib.fe2o3_prepared_patch_kernarg(self._h, C.c_uint64(offset), buf, C.c_uint64(len(data))), "patch_kernarg")

    @property
    def symbol(self):
        return lib.fe2o3_prepared_symbol(self._h).decode()

    def destroy(self):
        if self._h:
            lib.fe2o3_prepared_destroy(self._h)
            self._h = None


def make_args(op, **kw):
    cls = _lib.OPS[op][0]
    a = cls()
    for name, ty in cls._fields_:
        if name == "reserved":
            continue
        if name not in kw:
            if ty is Slice:
                setattr(a, name, Slice(0, 0))
            continue
        v = kw.pop(name)
        setattr(a, name, as_slice(v) if ty is Slice else v)
    if kw:
        raise TypeError(f"{op}: unknown arguments {sorted(kw)}")
    return a


def check_args(op, args):
    """Pure host admission (no CUDA call); raises Fe2o3Error on rejection."""
    check(getattr(lib, f"fe2o3_{op}_check")(C.byref(args)), f"{op}.check")


def prepare(ctx, op, schedule=SCHEDULE_AUTO, **kw):
    """`<kernel>_gpu::Kernel::load(ctx).prepare(...)` for the named op.

    Returns None when the plan is "empty output: nothing to dispatch"
    (examples/tiled_gemm_v1/src/contract.rs:401-407)."""
    args = make_args(op, **kw)
    h = C.c_void_p()
    fn = getattr(lib, f"fe2o3_{op}_prepare")
    if _lib.OPS[op][2]:
        st = fn(ctx._h, C.byref(args), C.c_uint32(schedule), C.byref(h))
    else:
        st = fn(ctx._h, C.byref(args), C.byref(h))
    if st == ERR_NO_DISPATCH:
        return None
    check(st, f"{op}.prepare")
    return Prepared(ctx, h, op)


def launch_count():
    return int(lib.fe2o3_launch_count())
