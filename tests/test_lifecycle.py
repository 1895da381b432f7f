"""One-shot lifecycle against a fake runtime adapter that substitutes one observation at a time.

Shape of crates/fe2o3-host/src/flash_attention_v1_lifecycle_tests.rs:22-56 (the Fault list) and
:444-592 (the four scenarios): exact event order, fail-closed on every substituted field, exactly one
unload on every path that loaded, leases released at quiescence only, kernel dropped before unload.
"""
import gc
import hashlib

import pytest

from fe2o3_b200 import lifecycle as lc

RUNTIME_INSTANCE = bytes([0x31]) * 16
AGENT_HANDLE = 0x5354
EXECUTABLE_OBJECT = bytes([0x65]) * 32
KERNEL_OBJECT = bytes([0x76]) * 32
DISPATCH_IDENTITY = bytes([0x87]) * 16
SYMBOL = "flash_attention_v1"
GEOMETRY = lc.Geometry((148, 1, 1), (384, 1, 1), 198144)
ARTIFACT = b"exact-finalized-FlashAttention-v1"
CONTEXT = hashlib.sha256(b"context").digest()

LOAD_FAULTS = ["EnvironmentAdapter", "EnvironmentTarget", "EnvironmentOrdinal", "LoadAdapter", "LoadDigest", "LoadLength",
               "LoadRuntime", "LoadAgent", "ResolveAdapter", "ResolutionExecutable", "ResolutionSymbol", "ResolutionSize",
               "ResolutionAlignment", "ResourceAdapter", "ResourceExecutable", "ResourceKernel", "ResourceGroup",
               "ResourcePrivate"]
NO_UNLOAD = {"EnvironmentAdapter", "EnvironmentTarget", "EnvironmentOrdinal", "LoadAdapter"}
DISPATCH_FAULTS = ["ImplicitAdapter", "ImplicitExecutable", "ImplicitKernel", "ImplicitGeometry", "ImplicitSpan",
                   "ImplicitIncomplete", "ExplicitMutation", "DispatchAdapter", "DispatchTimeout", "DispatchExecutable",
                   "DispatchKernel", "DispatchGeometry", "DispatchIncomplete", "DispatchKernelStatus"]


class Lease:
    def __init__(self, log):
        self.log = log

    def release(self):
        self.log.append("lease_drop")


class FakeKernel:
    def __init__(self, events):
        self.events, self.object = events, KERNEL_OBJECT

    def close(self):
        self.events.append("kernel_drop")


class FakeAdapter(lc.RuntimeAdapter):
    def __init__(self, fault=None):
        self.fault, self.events, self.unloads = fault, [], 0
        self.aligned = self.explicit_preserved = False

    def context_identity(self):
        return CONTEXT

    def observe_environment(self):
        self.events.append("environment")
        if self.fault == "EnvironmentAdapter":
            raise RuntimeError("environment")
        return lc.EnvironmentObservation("sm_90a" if self.fault == "EnvironmentTarget" else lc.TARGET,
                                         1 if self.fault == "EnvironmentOrdinal" else 0, RUNTIME_INSTANCE, AGENT_HANDLE)

    def load_executable(self, artifact_bytes, digest):
        self.events.append("load")
        if self.fault == "LoadAdapter":
            raise RuntimeError("load")
        assert artifact_bytes == ARTIFACT and digest == hashlib.sha256(ARTIFACT).digest()
        obs = lc.LoadObservation(bytes(32) if self.fault == "LoadDigest" else digest,
                                 len(artifact_bytes) - (self.fault == "LoadLength"),
                                 bytes(16) if self.fault == "LoadRuntime" else RUNTIME_INSTANCE,
                                 AGENT_HANDLE + (self.fault == "LoadAgent"), EXECUTABLE_OBJECT)
        return "executable", obs

    def resolve_kernel(self, executable, symbol):
        self.events.append("resolve")
        if self.fault == "ResolveAdapter":
            raise RuntimeError("resolve")
        obs = lc.ResolutionObservation(bytes([0xa1]) * 32 if self.fault == "ResolutionExecutable" else EXECUTABLE_OBJECT,
                                       "other" if self.fault == "ResolutionSymbol" else symbol, KERNEL_OBJECT,
                                       96 - (self.fault == "ResolutionSize"),
                                       8 if self.fault == "ResolutionAlignment" else lc.KERNARG_ALIGNMENT)
        return FakeKernel(self.events), obs

    def observe_kernel_resources(self, executable, kernel):
        self.events.append("resources")
        if self.fault == "ResourceAdapter":
            raise RuntimeError("resources")
        return lc.ResourceObservation(bytes([0xc1]) * 32 if self.fault == "ResourceExecutable" else EXECUTABLE_OBJECT,
                                      bytes([0xc2]) * 32 if self.fault == "ResourceKernel" else kernel.object,
                                      int(self.fault == "ResourceGroup"), int(self.fault == "ResourcePrivate"))

    def initialize_implicit_kernarg(self, executable, kernel, geometry, explicit_byte_len, implicit_byte_offset,
                                    implicit_byte_len, kernarg):
        import ctypes as C
        self.events.append("implicit")
        self.aligned = C.addressof(kernarg) % lc.KERNARG_ALIGNMENT == 0
        self.explicit_preserved = bytes(kernarg) == bytes(range(96))
        if self.fault == "ImplicitAdapter":
            raise RuntimeError("implicit")
        if self.fault == "ExplicitMutation":
            kernarg[0] ^= 1
        return lc.ImplicitKernargObservation(
            bytes([0xb1]) * 32 if self.fault == "ImplicitExecutable" else EXECUTABLE_OBJECT,
            bytes([0xb2]) * 32 if self.fault == "ImplicitKernel" else kernel.object,
            lc.Geometry((2, 1, 1), GEOMETRY.workgroup, 0) if self.fault == "ImplicitGeometry" else geometry,
            explicit_byte_len - (self.fault == "ImplicitSpan"), implicit_byte_offset, implicit_byte_len,
            self.fault != "ImplicitIncomplete")

    def launch_and_wait(self, executable, kernel, geometry, kernarg):
        self.events.append("dispatch")
        if self.fault == "DispatchAdapter":
            raise RuntimeError("dispatch")
        if self.fault == "DispatchTimeout":
            raise TimeoutError("ambiguous completion")
        return lc.DispatchObservation(
            bytes([0xd1]) * 32 if self.fault == "DispatchExecutable" else EXECUTABLE_OBJECT,
            bytes([0xd2]) * 32 if self.fault == "DispatchKernel" else kernel.object,
            lc.Geometry((2, 1, 1), GEOMETRY.workgroup, 0) if self.fault == "DispatchGeometry" else geometry,
            self.fault != "DispatchIncomplete", DISPATCH_IDENTITY, 2 if self.fault == "DispatchKernelStatus" else 0)

    def unload_executable(self, executable):
        self.events.append("unload")
        self.unloads += 1
        return lc.UnloadObservation(EXECUTABLE_OBJECT, True)


def receipt():
    content = lc.ContentIdentity.calculate(ARTIFACT)
    return lc.ArtifactReceipt(bytes([1]) * 32, content.digest, content, lc.TARGET, SYMBOL, ARTIFACT)


def joined(log, **kw):
    binding = lc.LaunchBinding(kw.get("symbol", SYMBOL), bytes(range(96)), kw.get("geometry", GEOMETRY), CONTEXT, 0,
                               leases=[Lease(log)], target=kw.get("target", lc.TARGET))
    return lc.join(kw.get("receipt", receipt()), binding)


def test_successful_exact_lifecycle_preserves_abi_and_releases_leases_at_quiescence():
    adapter, log = FakeAdapter(), []
    loaded = joined(log).load(adapter)
    assert log == [] and adapter.events == ["environment", "load", "resolve", "resources"]
    completed = loaded.dispatch_and_wait()
    assert adapter.aligned and adapter.explicit_preserved
    assert log == ["lease_drop"]                      # released at quiescence, before the unload
    assert adapter.unloads == 0
    done = completed.unload()
    assert adapter.unloads == 1
    assert adapter.events == ["environment", "load", "resolve", "resources", "implicit", "dispatch", "kernel_drop", "unload"]
    assert done.dispatch_identity == DISPATCH_IDENTITY and done.executable_object == EXECUTABLE_OBJECT
    assert done.kernel_object == KERNEL_OBJECT and done.receipt_identity == bytes([1]) * 32
    assert len(done.unload_identity) == 32 and done.dispatched_exact_structural_profile
    assert not done.proves_compiler_refinement and not done.proves_general_memory_safety_or_race_freedom


@pytest.mark.parametrize("fault", LOAD_FAULTS)
def test_every_load_and_resource_substitution_fails_closed_with_exact_cleanup(fault):
    adapter, log = FakeAdapter(fault), []
    with pytest.raises(lc.LoadError):
        joined(log).load(adapter)
    assert adapter.unloads == (0 if fault in NO_UNLOAD else 1), fault
    assert log == ["lease_drop"], fault
    if "unload" in adapter.events and "kernel_drop" in adapter.events:
        assert adapter.events.index("kernel_drop") < adapter.events.index("unload")


@pytest.mark.parametrize("fault", DISPATCH_FAULTS)
def test_implicit_dispatch_timeout_and_observation_failures_cleanup_once(fault):
    adapter, log = FakeAdapter(fault), []
    loaded = joined(log).load(adapter)
    with pytest.raises(lc.DispatchError):
        loaded.dispatch_and_wait()
    assert adapter.unloads == 1 and log == ["lease_drop"], fault
    assert adapter.events.index("kernel_drop") < adapter.events.index("unload"), adapter.events


def test_dropping_loaded_or_completed_state_unloads_exactly_once():
    adapter, log = FakeAdapter(), []
    loaded = joined(log).load(adapter)
    del loaded
    gc.collect()
    assert adapter.unloads == 1 and log == ["lease_drop"]
    adapter, log = FakeAdapter(), []
    completed = joined(log).load(adapter).dispatch_and_wait()
    del completed
    gc.collect()
    assert adapter.unloads == 1 and log == ["lease_drop"]
    adapter, log = FakeAdapter(), []
    joined(log).load(adapter).abandon()
    assert adapter.unloads == 1 and log == ["lease_drop"]


def test_states_are_one_shot():
    adapter, log = FakeAdapter(), []
    j = joined(log)
    loaded = j.load(adapter)
    with pytest.raises(lc.ConsumedError):
        j.load(adapter)
    completed = loaded.dispatch_and_wait()
    with pytest.raises(lc.ConsumedError):
        loaded.dispatch_and_wait()
    completed.unload()
    with pytest.raises(lc.ConsumedError):
        completed.unload()
    assert adapter.unloads == 1


def test_context_identity_mismatch_is_refused_before_any_adapter_observation():
    adapter, log = FakeAdapter(), []
    adapter.context_identity = lambda: hashlib.sha256(b"another context").digest()
    with pytest.raises(lc.LoadError) as err:
        joined(log).load(adapter)
    assert err.value.kind == "ContextIdentity" and str(err.value) == "exact CUDA context identity mismatch"
    assert adapter.events == [] and log == ["lease_drop"]


def test_join_rejects_receipts_and_bindings_that_do_not_agree():
    content = lc.ContentIdentity.calculate(ARTIFACT)
    bad_receipts = {
        "identity": lc.ArtifactReceipt(bytes(32), content.digest, content, lc.TARGET, SYMBOL, ARTIFACT),
        "artifact identity": lc.ArtifactReceipt(bytes([1]) * 32, bytes(32), content, lc.TARGET, SYMBOL, ARTIFACT),
        "finalized output": lc.ArtifactReceipt(bytes([1]) * 32, content.digest, lc.ContentIdentity(content.digest, 0),
                                               lc.TARGET, SYMBOL, ARTIFACT),
        "target": lc.ArtifactReceipt(bytes([1]) * 32, content.digest, content, "gfx942", SYMBOL, ARTIFACT),
        "symbol": lc.ArtifactReceipt(bytes([1]) * 32, content.digest, content, lc.TARGET, "row_softmax_v1", ARTIFACT),
    }
    for field, r in bad_receipts.items():
        with pytest.raises(lc.JoinError) as err:
            joined([], receipt=r)
        assert err.value.field == field
    with pytest.raises(lc.JoinError):
        joined([], geometry=lc.Geometry((0, 1, 1), (384, 1, 1), 0))


def test_tampered_artifact_bytes_never_reach_the_adapter():
    content = lc.ContentIdentity.calculate(ARTIFACT)
    r = lc.ArtifactReceipt(bytes([1]) * 32, content.digest, content, lc.TARGET, SYMBOL, ARTIFACT[:-1] + b"2")
    adapter, log = FakeAdapter(), []
    with pytest.raises(lc.LoadError) as err:
        joined(log, receipt=r).load(adapter)
    assert err.value.kind == "FinalizedOutput" and "load" not in adapter.events and adapter.unloads == 0
