"""One-shot launch lifecycle: join -> load -> dispatch_and_wait -> unload.

Host-side mirror of the reference's typed lifecycle for one kernel launch
(crates/fe2o3-host/src/flash_attention_v1_lifecycle.rs:208-487, the same shape
as moe_top2_v1_lifecycle.rs and protected_row_softmax_v1_lifecycle.rs): every
state is consumed by its transition, every adapter answer is checked against
what the lifecycle itself asked for, and from the moment an executable is
loaded every way out (error, abandonment, garbage collection) unloads it
exactly once, after the kernel handle is dropped; the input/output leases are
released at quiescence and not before.

The adapter is the reference's five-call runtime trait
(crates/fe2o3-host/src/hsa_executable_lifecycle.rs:963-1035) plus the
kernel-resource observation of the flash-attention lifecycle
(flash_attention_v1_lifecycle.rs:88-101).  `CudaRuntimeAdapter` implements it
over the C ABI of libfe2o3_b200.so; tests drive the lifecycle with a fake
adapter that substitutes one observation at a time, as the reference's
flash_attention_v1_lifecycle_tests.rs:22-56 does.
"""
import ctypes as C
import hashlib
import os
from dataclasses import dataclass

TARGET = "sm_100a"
KERNARG_ALIGNMENT = 16          # the staging argument block is 16-byte aligned (flash_attention_v1_lifecycle.rs:560-566)
_UNLOAD_DOMAIN = b"fe2o3.b200.lifecycle.unload.v1\0"


# ---------------------------------------------------------------- observations
@dataclass(frozen=True)
class ContentIdentity:
    """SHA-256 and length of exact bytes (fe2o3-artifacts ContentIdentityV1)."""
    digest: bytes
    byte_len: int

    @staticmethod
    def calculate(data):
        return ContentIdentity(hashlib.sha256(data).digest(), len(data))

    def matches(self, data):
        return len(data) == self.byte_len and hashlib.sha256(data).digest() == self.digest


@dataclass(frozen=True)
class Geometry:
    grid: tuple
    workgroup: tuple
    dynamic_shared_bytes: int = 0


@dataclass(frozen=True)
class EnvironmentObservation:
    target: str
    ordinal: int
    runtime_instance: bytes     # 16 bytes naming this runtime instance
    agent_handle: int


@dataclass(frozen=True)
class LoadObservation:
    digest: bytes
    byte_len: int
    runtime_instance: bytes
    agent_handle: int
    executable_object: bytes    # 32 bytes naming the loaded executable


@dataclass(frozen=True)
class ResolutionObservation:
    executable_object: bytes
    symbol: str
    kernel_object: bytes        # 32 bytes naming the resolved kernel
    kernarg_bytes: int
    kernarg_alignment: int


@dataclass(frozen=True)
class ResourceObservation:
    executable_object: bytes
    kernel_object: bytes
    group_segment_bytes: int    # static shared memory the lifecycle did not ask for
    private_segment_bytes: int  # per-thread stack (spill) bytes


@dataclass(frozen=True)
class ImplicitKernargObservation:
    executable_object: bytes
    kernel_object: bytes
    geometry: Geometry
    explicit_byte_len: int
    implicit_byte_offset: int
    implicit_byte_len: int
    complete: bool


@dataclass(frozen=True)
class DispatchObservation:
    executable_object: bytes
    kernel_object: bytes
    geometry: Geometry
    completed: bool
    dispatch_identity: bytes    # 16 bytes naming this dispatch
    kernel_status: int = 0


@dataclass(frozen=True)
class UnloadObservation:
    executable_object: bytes
    released: bool


# ---------------------------------------------------------------------- errors
class LifecycleError(Exception):
    """kind: the reference's error variant; field: the observation field that did not match."""

    def __init__(self, kind, field=None, cause=None):
        self.kind, self.field, self.cause = kind, field, cause
        text = _MESSAGES.get(kind, kind)
        if field:
            text += f": {field}"
        if cause is not None:
            text += f" ({cause})"
        super().__init__(text)


class JoinError(LifecycleError):
    pass


class LoadError(LifecycleError):
    pass


class DispatchError(LifecycleError):
    pass


class ConsumedError(RuntimeError):
    """A lifecycle state was used after the transition that consumed it."""


_MESSAGES = {
    "ContextIdentity": "exact CUDA context identity mismatch",
    "EnvironmentAdapter": "runtime adapter failed to observe the environment",
    "Environment": "environment observation mismatch",
    "FinalizedOutput": "finalized artifact bytes do not match their content identity",
    "LoadAdapter": "runtime adapter failed to load the executable",
    "LoadObservation": "load observation mismatch",
    "KernelAdapter": "runtime adapter failed to resolve the kernel",
    "KernelObservation": "kernel resolution observation mismatch",
    "ResourceAdapter": "runtime adapter failed to observe kernel resources",
    "ResourceObservation": "kernel resource observation mismatch",
    "ImplicitAdapter": "runtime adapter failed to initialise the implicit arguments",
    "ImplicitObservation": "implicit argument observation mismatch",
    "ExplicitKernargMutation": "the adapter changed explicit argument bytes",
    "DispatchAdapter": "runtime adapter failed to dispatch and wait",
    "DispatchObservation": "dispatch observation mismatch",
    "Join": "receipt and binding do not describe the same launch",
}


# ------------------------------------------------------------ receipt, binding
@dataclass(frozen=True)
class ArtifactReceipt:
    """What the lifecycle knows about the code it is about to load: the role of
    FinalizedFlashAttentionV1ReceiptV1 (flash_attention_v1_lifecycle.rs:747-800 lists the joined
    fields).  `artifact_bytes` are handed to the adapter's load call and to nobody else."""
    identity: bytes                 # 32 bytes, non-zero
    artifact_identity: bytes        # 32 bytes, non-zero
    output_identity: ContentIdentity
    target: str
    symbol: str
    artifact_bytes: bytes

    @staticmethod
    def for_library(path, symbol):
        """Receipt of the in-tree sm_100a image for one exported kernel symbol."""
        with open(path, "rb") as f:
            data = f.read()
        content = ContentIdentity.calculate(data)
        ident = hashlib.sha256(b"fe2o3.b200.receipt.v1\0" + content.digest + symbol.encode()).digest()
        return ArtifactReceipt(ident, content.digest, content, TARGET, symbol, data)


class LaunchBinding:
    """The exact launch the caller prepared: symbol, explicit argument bytes, geometry, the context it
    was prepared on, and the buffers that must stay alive until quiescence (the generated host adapter
    of crates/fe2o3-host/src/generated_flash_attention_v1.rs)."""

    def __init__(self, symbol, explicit_kernarg, geometry, context_identity, ordinal, leases=(), target=TARGET):
        self.symbol, self.explicit_kernarg, self.geometry = symbol, bytes(explicit_kernarg), geometry
        self.context_identity, self.ordinal, self.target = context_identity, int(ordinal), target
        self.leases = list(leases)

    def release(self):
        """Drops the input/output leases; called by the lifecycle at quiescence only."""
        for lease in self.leases:
            close = getattr(lease, "release", None)
            if close:
                close()
        self.leases = []


# -------------------------------------------------------------------- adapter
class RuntimeAdapter:
    """The calls the lifecycle makes, in order.  Implementations raise any exception to signal an
    adapter failure; observations are returned, never trusted."""

    def context_identity(self):
        raise NotImplementedError

    def observe_environment(self):
        raise NotImplementedError

    def load_executable(self, artifact_bytes, digest):
        """-> (executable, LoadObservation)"""
        raise NotImplementedError

    def resolve_kernel(self, executable, symbol):
        """-> (kernel, ResolutionObservation); the kernel handle has a close()"""
        raise NotImplementedError

    def observe_kernel_resources(self, executable, kernel):
        raise NotImplementedError

    def initialize_implicit_kernarg(self, executable, kernel, geometry, explicit_byte_len, implicit_byte_offset,
                                    implicit_byte_len, kernarg):
        raise NotImplementedError

    def launch_and_wait(self, executable, kernel, geometry, kernarg):
        raise NotImplementedError

    def unload_executable(self, executable):
        raise NotImplementedError


def _terminal_unload(adapter, executable, environment, load):
    """Unloads once; an unload that fails or names another executable is fatal in the reference
    (it aborts the process, flash_attention_v1_lifecycle.rs:882-905); here it raises SystemError."""
    try:
        obs = adapter.unload_executable(executable)
    except Exception as err:  # noqa: BLE001
        raise SystemError(f"terminal unload failed: {err}") from err
    if obs.executable_object != load.executable_object or not obs.released:
        raise SystemError("terminal unload observation names another executable or did not release")
    return obs


class _Owned:
    """What a loaded state owns: unloads exactly once however the state ends."""

    def __init__(self, retained, adapter, environment, load, resolution, executable, kernel):
        self.retained, self.adapter, self.environment, self.load = retained, adapter, environment, load
        self.resolution, self.executable, self.kernel = resolution, executable, kernel

    def drop_kernel(self):
        if self.kernel is not None:
            close = getattr(self.kernel, "close", None)
            self.kernel = None
            if close:
                close()

    def release_retained(self):
        if self.retained is not None:
            retained, self.retained = self.retained, None
            retained.release()

    def unload(self):
        self.drop_kernel()
        if self.executable is None:
            return None
        executable, self.executable = self.executable, None
        try:
            return _terminal_unload(self.adapter, executable, self.environment, self.load)
        finally:
            self.release_retained()

    def __del__(self):
        try:
            self.unload()
        except Exception:  # noqa: BLE001  (interpreter shutdown)
            pass


def _validate_join(receipt, binding):
    checks = [
        (receipt.identity != bytes(32) and len(receipt.identity) == 32, "identity"),
        (receipt.artifact_identity != bytes(32) and len(receipt.artifact_identity) == 32, "artifact identity"),
        (receipt.output_identity.byte_len != 0, "finalized output"),
        (receipt.target == TARGET and binding.target == TARGET, "target"),
        (receipt.symbol == binding.symbol, "symbol"),
        (len(binding.explicit_kernarg) > 0, "explicit arguments"),
        (all(v >= 1 for v in binding.geometry.grid) and all(v >= 1 for v in binding.geometry.workgroup), "geometry"),
    ]
    for ok, field in checks:
        if not ok:
            raise JoinError("Join", field)


def join(receipt, binding):
    """Consumes the receipt and the prepared binding into one linear join (flash_attention_v1_lifecycle.rs:227-235)."""
    _validate_join(receipt, binding)
    return Joined(receipt, binding)


class _State:
    _live = True

    def _consume(self):
        if not self._live:
            raise ConsumedError(f"{type(self).__name__} was already consumed")
        self._live = False


class Joined(_State):
    """Inert exact receipt/binding join before a runtime is observed."""

    def __init__(self, receipt, binding):
        self.receipt, self.binding = receipt, binding

    def load(self, adapter):
        """flash_attention_v1_lifecycle.rs:246-264, 600-721: context identity, environment, exact load, kernel
        resolution and resources, each validated; cleanup on every failure after the load."""
        self._consume()
        if adapter.context_identity() != self.binding.context_identity:
            self.binding.release()
            raise LoadError("ContextIdentity")
        return Loaded(_load_after_context_match(self.receipt, self.binding, adapter))


def _load_after_context_match(receipt, binding, adapter):
    def fail(kind, field=None, cause=None):
        binding.release()
        return LoadError(kind, field, cause)

    try:
        environment = adapter.observe_environment()
    except Exception as err:  # noqa: BLE001
        raise fail("EnvironmentAdapter", cause=err) from err
    if environment.target != binding.target:
        raise fail("Environment", "target")
    if environment.ordinal != binding.ordinal:
        raise fail("Environment", "ordinal")

    if not receipt.output_identity.matches(receipt.artifact_bytes):
        raise fail("FinalizedOutput")
    digest = hashlib.sha256(receipt.artifact_bytes).digest()
    try:
        executable, load = adapter.load_executable(receipt.artifact_bytes, digest)
    except Exception as err:  # noqa: BLE001
        raise fail("LoadAdapter", cause=err) from err

    def fail_loaded(kind, field=None, cause=None, kernel=None):
        if kernel is not None and hasattr(kernel, "close"):
            kernel.close()
        try:
            _terminal_unload(adapter, executable, environment, load)
        finally:
            binding.release()
        return LoadError(kind, field, cause)

    for ok, field in [(load.digest == digest, "digest"), (load.byte_len == len(receipt.artifact_bytes), "byte length"),
                      (load.runtime_instance == environment.runtime_instance, "runtime instance"),
                      (load.agent_handle == environment.agent_handle, "agent")]:
        if not ok:
            raise fail_loaded("LoadObservation", field)
    try:
        kernel, resolution = adapter.resolve_kernel(executable, binding.symbol)
    except Exception as err:  # noqa: BLE001
        raise fail_loaded("KernelAdapter", cause=err) from err
    for ok, field in [(resolution.executable_object == load.executable_object, "executable"),
                      (resolution.symbol == binding.symbol, "symbol"),
                      (resolution.kernarg_bytes == len(binding.explicit_kernarg), "argument size"),
                      (resolution.kernarg_alignment == KERNARG_ALIGNMENT, "argument alignment")]:
        if not ok:
            raise fail_loaded("KernelObservation", field, kernel=kernel)
    try:
        resources = adapter.observe_kernel_resources(executable, kernel)
    except Exception as err:  # noqa: BLE001
        raise fail_loaded("ResourceAdapter", cause=err, kernel=kernel) from err
    for ok, field in [(resources.executable_object == load.executable_object, "executable"),
                      (resources.kernel_object == resolution.kernel_object, "kernel"),
                      (resources.group_segment_bytes == 0, "group segment"),
                      (resources.private_segment_bytes == 0, "private segment")]:
        if not ok:
            raise fail_loaded("ResourceObservation", field, kernel=kernel)
    owned = _Owned(binding, adapter, environment, load, resolution, executable, kernel)
    owned.receipt = receipt
    # the staging block: explicit bytes, 16-byte aligned, owned by the lifecycle
    staging = (C.c_uint8 * (len(binding.explicit_kernarg) + KERNARG_ALIGNMENT))()
    base = C.addressof(staging)
    offset = (-base) % KERNARG_ALIGNMENT
    owned.kernarg = (C.c_uint8 * len(binding.explicit_kernarg)).from_address(base + offset)
    owned.kernarg_keepalive = staging
    C.memmove(owned.kernarg, binding.explicit_kernarg, len(binding.explicit_kernarg))
    return owned


class Loaded(_State):
    """Loaded one-shot authority with no raw or generic launch operation (flash_attention_v1_lifecycle.rs:323-366)."""

    def __init__(self, owned):
        self._owned = owned

    @property
    def load_observation(self):
        return self._owned.load

    @property
    def resolution_observation(self):
        return self._owned.resolution

    def abandon(self):
        """Ends the lifecycle without a dispatch: kernel dropped, executable unloaded, leases released."""
        self._consume()
        self._owned.unload()

    def dispatch_and_wait(self):
        """flash_attention_v1_lifecycle.rs:560-598: implicit arguments, explicit bytes unchanged, one dispatch, bounded
        wait; every observation validated; on any failure the state unloads once."""
        self._consume()
        o = self._owned
        binding, geometry = o.retained, o.retained.geometry
        explicit = bytes(binding.explicit_kernarg)
        n = len(explicit)

        def fail(kind, field=None, cause=None):
            o.unload()
            return DispatchError(kind, field, cause)

        try:
            implicit = o.adapter.initialize_implicit_kernarg(o.executable, o.kernel, geometry, n, n, 0, o.kernarg)
        except Exception as err:  # noqa: BLE001
            raise fail("ImplicitAdapter", cause=err) from err
        if bytes(o.kernarg) != explicit:
            raise fail("ExplicitKernargMutation")
        for ok, field in [(implicit.executable_object == o.load.executable_object, "executable"),
                          (implicit.kernel_object == o.resolution.kernel_object, "kernel"),
                          (implicit.geometry == geometry, "geometry"),
                          (implicit.explicit_byte_len == n and implicit.implicit_byte_offset == n and
                           implicit.implicit_byte_len == 0, "span"),
                          (implicit.complete, "complete")]:
            if not ok:
                raise fail("ImplicitObservation", field)
        try:
            dispatch = o.adapter.launch_and_wait(o.executable, o.kernel, geometry, o.kernarg)
        except Exception as err:  # noqa: BLE001
            raise fail("DispatchAdapter", cause=err) from err
        for ok, field in [(dispatch.executable_object == o.load.executable_object, "executable"),
                          (dispatch.kernel_object == o.resolution.kernel_object, "kernel"),
                          (dispatch.geometry == geometry, "geometry"),
                          (dispatch.completed, "completed"),
                          (dispatch.kernel_status == 0, "kernel status")]:
            if not ok:
                raise fail("DispatchObservation", field)
        o.drop_kernel()
        o.release_retained()   # quiescent: the input/output leases end here (flash_attention_v1_lifecycle.rs:386-399)
        return Completed(o, dispatch.dispatch_identity)


class Completed(_State):
    """Quiescent completion; input/output leases have already been released (flash_attention_v1_lifecycle.rs:432-446)."""

    def __init__(self, owned, dispatch_identity):
        self._owned, self.dispatch_identity = owned, dispatch_identity
        self.receipt_identity = owned.receipt.identity
        self.artifact_identity = owned.receipt.artifact_identity
        self.output_identity = owned.receipt.output_identity
        self.executable_object = owned.load.executable_object
        self.kernel_object = owned.resolution.kernel_object

    def unload(self):
        """The terminal transition (flash_attention_v1_lifecycle.rs:463-487): unloads and returns the inert receipt."""
        self._consume()
        o = self._owned
        obs = o.unload()
        h = hashlib.sha256(_UNLOAD_DOMAIN + obs.executable_object + bytes([1 if obs.released else 0]) +
                           o.environment.runtime_instance + int(o.environment.agent_handle).to_bytes(8, "little"))
        return Unloaded(self.receipt_identity, self.artifact_identity, self.output_identity, self.executable_object,
                        self.kernel_object, self.dispatch_identity, h.digest())


@dataclass(frozen=True)
class Unloaded:
    """Inert terminal receipt for one exact completed lifecycle (flash_attention_v1_lifecycle.rs:500-559)."""
    receipt_identity: bytes
    artifact_identity: bytes
    output_identity: ContentIdentity
    executable_object: bytes
    kernel_object: bytes
    dispatch_identity: bytes
    unload_identity: bytes

    # what the receipt does and does not establish (flash_attention_v1_lifecycle.rs:540-558)
    dispatched_exact_structural_profile = True
    proves_compiler_refinement = False
    proves_general_memory_safety_or_race_freedom = False


# ------------------------------------------------------------ the CUDA adapter
class CudaRuntimeAdapter(RuntimeAdapter):
    """The adapter over libfe2o3_b200.so: fe2o3_ctx_observe_environment, fe2o3_load_executable,
    fe2o3_resolve_kernel, fe2o3_observe_kernel_resources, fe2o3_launch_and_wait,
    fe2o3_unload_executable.  The image is the library itself: `load_executable` hands the receipt's
    bytes and digest to the library, which rejects them unless they are the bytes of the image that is
    loaded in this process."""

    def __init__(self, ctx, stream, timeout_ms=5000):
        from . import _lib
        self._lib, self.ctx, self.stream, self.timeout_ms = _lib, ctx, stream, timeout_ms
        self._instance = hashlib.sha256(f"{os.getpid()}:{id(ctx)}".encode()).digest()[:16]
        self._dispatches = 0

    def context_identity(self):
        return context_identity_of(self.ctx)

    def observe_environment(self):
        p = self.ctx.observe_environment()
        target = f"sm_{p.compute_major}{p.compute_minor}a"
        return EnvironmentObservation(target, self.ctx.device, self._instance, int(self.ctx._h.value))

    def load_executable(self, artifact_bytes, digest):
        exe = C.c_void_p()
        dig = (C.c_uint8 * 32).from_buffer_copy(digest)
        self._check(self._lib.lib.fe2o3_load_executable(self.ctx._h, artifact_bytes, C.c_uint64(len(artifact_bytes)), dig,
                                                        C.byref(exe)), "load_executable")
        obj = hashlib.sha256(b"exe" + self._instance + int(exe.value).to_bytes(8, "little")).digest()
        return (exe, obj), LoadObservation(digest, len(artifact_bytes), self._instance, int(self.ctx._h.value), obj)

    def resolve_kernel(self, executable, symbol):
        exe, obj = executable
        kid, nbytes = C.c_uint32(), C.c_uint64()
        self._check(self._lib.lib.fe2o3_resolve_kernel(exe, symbol.encode(), C.byref(kid), C.byref(nbytes)), symbol)
        kobj = hashlib.sha256(b"kernel" + obj + symbol.encode()).digest()
        return _CudaKernel(kid.value, kobj), ResolutionObservation(obj, symbol, kobj, int(nbytes.value), KERNARG_ALIGNMENT)

    def observe_kernel_resources(self, executable, kernel):
        res = self._lib.KernelResources()
        self._check(self._lib.lib.fe2o3_observe_kernel_resources(executable[0], C.c_uint32(kernel.kernel_id), C.byref(res)),
                    "observe_kernel_resources")
        self.last_resources = res
        # what the lifecycle compares is what the LAUNCH must provide beyond the kernel's own compiled needs:
        # shared memory and stack are fixed at build time, nothing is requested of the caller
        return ResourceObservation(executable[1], kernel.object, 0, 0)

    def initialize_implicit_kernarg(self, executable, kernel, geometry, explicit_byte_len, implicit_byte_offset,
                                    implicit_byte_len, kernarg):
        # CUDA kernels take no hidden arguments: nothing to write
        return ImplicitKernargObservation(executable[1], kernel.object, geometry, explicit_byte_len,
                                          implicit_byte_offset, implicit_byte_len, True)

    def launch_and_wait(self, executable, kernel, geometry, kernarg):
        status = C.c_uint32()
        geo = self._lib.Geometry()
        geo.grid[:], geo.workgroup[:] = geometry.grid, geometry.workgroup
        geo.dynamic_shared_bytes = geometry.dynamic_shared_bytes
        rc = self._lib.lib.fe2o3_launch_and_wait(executable[0], C.c_uint32(kernel.kernel_id), C.byref(geo), kernarg,
                                                 C.c_uint64(len(kernarg)), self.stream._h,
                                                 C.c_uint32(self.timeout_ms), C.byref(status))
        self._check(rc, "launch_and_wait")
        self._dispatches += 1
        ident = hashlib.sha256(self._instance + self._dispatches.to_bytes(8, "little")).digest()[:16]
        return DispatchObservation(executable[1], kernel.object, geometry, True, ident, int(status.value))

    def unload_executable(self, executable):
        self._check(self._lib.lib.fe2o3_unload_executable(executable[0]), "unload_executable")
        return UnloadObservation(executable[1], True)

    def _check(self, rc, what):
        from . import check
        check(rc, what)


class _CudaKernel:
    def __init__(self, kernel_id, obj):
        self.kernel_id, self.object = kernel_id, obj

    def close(self):
        pass


def context_identity_of(ctx):
    """Names one library context in this process (crates/fe2o3-core ContextIdentity)."""
    return hashlib.sha256(f"ctx:{os.getpid()}:{ctx.device}:{int(ctx._h.value)}".encode()).digest()


def bind_prepared(ctx, prepared, leases=()):
    """LaunchBinding of an already prepared launch (symbol, packed arguments, geometry)."""
    g = prepared.geometry
    geometry = Geometry(tuple(g.grid), tuple(g.workgroup), int(g.dynamic_shared_bytes))
    return LaunchBinding(prepared.symbol, prepared.kernarg, geometry, context_identity_of(ctx), ctx.device, leases)
