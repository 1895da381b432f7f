"""Runtime-neutral dispatch and wait records with the reference's canonical identity preimages.

The dispatch and wait flows of crates/fe2o3-host-api: operation context, resource bindings,
completion dependencies, the dispatch request and its result, the bounded wait request over
completion signals and its result (src/wait.rs:17-359), with the same structural
validation and the same bytes in `encode_identity_preimage()` (magic "F2HOSTP1",
little-endian, domain-separated; crates/fe2o3-host-api/src/canonical.rs:7-65,
src/dispatch.rs:234-268 and :350-368, src/common.rs:331-341, :495-500, :580-586), so a run
log written by a host that launches through this library hashes to the identities a
reference-side reader computes.  Records are inert descriptions: they own no runtime
handle and nothing here talks to a device.

All five flows of the crate are mirrored as records: compile (src/compile.rs), admit
(src/admit.rs), load (src/load.rs), dispatch and wait, together with the per-operation state chain (src/state.rs) and the
state-transition events and event batches (src/event.rs).
"""
import hashlib
from dataclasses import dataclass, field
from typing import Optional, Tuple

PREIMAGE_MAGIC_V1 = b"F2HOSTP1"
HOST_API_SCHEMA_VERSION_V1 = 1                     # src/lib.rs:48
IDENTITY_BYTES_V1 = 32                             # src/identity.rs:4
MAX_DIAGNOSTICS_V1 = 64                            # src/common.rs:18-26
MAX_DIAGNOSTIC_MESSAGE_BYTES_V1 = 1024
MAX_CAUSAL_EVENTS_V1 = 64
MAX_IDENTITY_PREIMAGE_BYTES_V1 = 128 * 1024
MAX_DISPATCH_BINDINGS_V1 = 128                     # src/dispatch.rs:19-22
MAX_DISPATCH_DEPENDENCIES_V1 = 128
MAX_WAIT_TARGETS_V1 = 256                          # src/wait.rs:17
MAX_PAYLOAD_BYTES_V1 = 256 * 1024 * 1024           # src/common.rs:17
MAX_ADMISSION_CLAIMS_V1 = 128                      # src/admit.rs:17
MAX_EVENT_BATCH_V1 = 512                           # src/event.rs:17

# identity domains used by the dispatch flow (src/identity.rs:55-272)
DOMAINS = {
    "FlowScopeId": b"fe2o3.host.scope.v1",
    "OperationId": b"fe2o3.host.operation.v1",
    "LoadedObjectId": b"fe2o3.host.loaded-object.v1",
    "EntryPointId": b"fe2o3.host.entry-point.v1",
    "ArgumentSetId": b"fe2o3.host.argument-set.v1",
    "DispatchContractId": b"fe2o3.host.dispatch-contract.v1",
    "ServiceInstanceId": b"fe2o3.host.service-instance.v1",
    "TaskSchemaId": b"fe2o3.host.task-schema.v1",
    "ResourceId": b"fe2o3.host.resource.v1",
    "DispatchSubmissionId": b"fe2o3.host.dispatch-submission.v1",
    "CompletionSignalId": b"fe2o3.host.completion-signal.v1",
    "LoadResultId": b"fe2o3.host.load.result.v1",
    "DispatchRequestId": b"fe2o3.host.dispatch.request.v1",
    "DispatchResultId": b"fe2o3.host.dispatch.result.v1",
    "PayloadId": b"fe2o3.host.payload.v1",
    "PayloadFormatId": b"fe2o3.host.payload-format.v1",
    "CompilerProfileId": b"fe2o3.host.compiler-profile.v1",
    "TargetProfileId": b"fe2o3.host.target-profile.v1",
    "CompileConfigurationId": b"fe2o3.host.compile-configuration.v1",
    "AdmissionPolicyId": b"fe2o3.host.admission-policy.v1",
    "ClaimId": b"fe2o3.host.claim.v1",
    "AdmissionAssessmentId": b"fe2o3.host.admission-assessment.v1",
    "LoaderProfileId": b"fe2o3.host.loader-profile.v1",
    "RuntimeContextId": b"fe2o3.host.runtime-context.v1",
    "CompileRequestId": b"fe2o3.host.compile.request.v1",
    "CompileResultId": b"fe2o3.host.compile.result.v1",
    "AdmitRequestId": b"fe2o3.host.admit.request.v1",
    "AdmitResultId": b"fe2o3.host.admit.result.v1",
    "LoadRequestId": b"fe2o3.host.load.request.v1",
    "CompletionRecordId": b"fe2o3.host.completion-record.v1",
    "DeadlineId": b"fe2o3.host.deadline.v1",
    "WaitRequestId": b"fe2o3.host.wait.request.v1",
    "WaitResultId": b"fe2o3.host.wait.result.v1",
    "CompileEventId": b"fe2o3.host.compile.event.v1",
    "AdmitEventId": b"fe2o3.host.admit.event.v1",
    "LoadEventId": b"fe2o3.host.load.event.v1",
    "DispatchEventId": b"fe2o3.host.dispatch.event.v1",
    "WaitEventId": b"fe2o3.host.wait.event.v1",
}

FLOW_COMPILE, FLOW_ADMIT, FLOW_LOAD, FLOW_DISPATCH, FLOW_WAIT = 1, 2, 3, 4, 5          # src/common.rs:165-176
ACCESS_READ, ACCESS_WRITE, ACCESS_READ_WRITE, ACCESS_ATOMIC = 1, 2, 3, 4               # src/common.rs:506-515
SEVERITY_NOTE, SEVERITY_WARNING, SEVERITY_ERROR = 1, 2, 3                              # src/common.rs:405-412


class HostContractError(ValueError):
    """kind: the reference's HostContractErrorV1 variant; field: its ContractFieldV1."""

    def __init__(self, kind, field=None):
        self.kind, self.field = kind, field
        super().__init__(f"{kind}({field})" if field else kind)


def digest(value):
    """A 32-byte commitment (HostDigestV1: width is checked, nothing is hashed or authenticated)."""
    b = bytes(value)
    if len(b) != IDENTITY_BYTES_V1:
        raise ValueError("a host digest is 32 bytes")
    return b


class Encoder:
    """canonical.rs:9-65: magic, u16 domain length, domain, u16 schema version, then fields little-endian."""

    def __init__(self, domain):
        self.bytes = bytearray(PREIMAGE_MAGIC_V1)
        self.u16(len(domain))
        self.bytes += domain
        self.u16(HOST_API_SCHEMA_VERSION_V1)

    def u8(self, v):
        self.bytes += int(v).to_bytes(1, "little")

    def u16(self, v):
        self.bytes += (int(v) & 0xffff).to_bytes(2, "little")

    def u32(self, v):
        self.bytes += int(v).to_bytes(4, "little")

    def u64(self, v):
        self.bytes += int(v).to_bytes(8, "little")

    def digest(self, d):
        self.bytes += digest(d)

    def optional_digest(self, d):
        if d is None:
            self.u8(0)
        else:
            self.u8(1)
            self.digest(d)

    def text(self, s):
        raw = s.encode("utf-8")
        self.u16(len(raw))
        self.bytes += raw

    def finish(self):
        assert len(self.bytes) <= MAX_IDENTITY_PREIMAGE_BYTES_V1
        return bytes(self.bytes)


def _strictly_ordered(values, maximum, fld):
    """common.rs:666-687."""
    if len(values) > maximum:
        raise HostContractError("TooManyItems", fld)
    for a, b in zip(values, values[1:]):
        if a == b:
            raise HostContractError("Duplicate", fld)
        if a > b:
            raise HostContractError("NonCanonicalOrder", fld)


@dataclass(frozen=True)
class OperationContext:
    """common.rs:265-342.  causal_events: (flow, 32-byte event identity), strictly increasing."""
    scope_id: bytes
    operation_id: bytes
    attempt: int
    parent_operation_id: Optional[bytes] = None
    causal_events: Tuple[Tuple[int, bytes], ...] = ()

    def __post_init__(self):
        digest(self.scope_id), digest(self.operation_id)
        if self.attempt == 0:
            raise HostContractError("Empty", "OperationAttempt")
        if not 0 < self.attempt < 1 << 16:
            raise ValueError("attempt is a u16")
        if self.parent_operation_id is not None and digest(self.parent_operation_id) == self.operation_id:
            raise HostContractError("Mismatch", "ParentOperation")
        events = [(int(f), digest(d)) for f, d in self.causal_events]
        _strictly_ordered(events, MAX_CAUSAL_EVENTS_V1, "CausalEvents")

    def encode(self, e):
        e.digest(self.scope_id)
        e.digest(self.operation_id)
        e.u16(self.attempt)
        e.optional_digest(self.parent_operation_id)
        e.u16(len(self.causal_events))
        for flow, ident in self.causal_events:
            e.u8(flow)
            e.digest(ident)


@dataclass(frozen=True)
class ResourceBinding:
    """common.rs:517-587: one resource range bound to an argument ordinal."""
    ordinal: int
    resource_identity: bytes
    access: int
    byte_offset: int
    byte_len: int

    def __post_init__(self):
        digest(self.resource_identity)
        if self.access not in (ACCESS_READ, ACCESS_WRITE, ACCESS_READ_WRITE, ACCESS_ATOMIC):
            raise ValueError("unknown access mode")
        if self.byte_len == 0:
            raise HostContractError("Empty", "ResourceRange")
        if self.byte_offset + self.byte_len >= 1 << 64:
            raise HostContractError("ArithmeticOverflow", "ResourceRange")

    def encode(self, e):
        e.u16(self.ordinal)
        e.digest(self.resource_identity)
        e.u8(self.access)
        e.u64(self.byte_offset)
        e.u64(self.byte_len)


@dataclass(frozen=True, order=True)
class DispatchDependency:
    """dispatch.rs:24-57: a predecessor completion this dispatch waits for."""
    completion_signal_identity: bytes
    producer_submission_identity: bytes

    def encode(self, e):
        e.digest(self.completion_signal_identity)
        e.digest(self.producer_submission_identity)


@dataclass(frozen=True)
class PersistentTask:
    """dispatch.rs:64-75."""
    service_instance_identity: bytes
    task_schema_identity: bytes
    task_tag: int
    service_epoch: int


@dataclass(frozen=True)
class LoadedResult:
    """What a dispatch request copies from a successful load result (load.rs LoadOutcomeV1::Loaded)."""
    identity: bytes
    loaded_object_identity: bytes
    load_generation: int


@dataclass(frozen=True)
class Diagnostic:
    """common.rs:446-500."""
    code: int
    severity: int
    message: str
    subject: Optional[bytes] = None

    def __post_init__(self):
        if self.code == 0:
            raise HostContractError("Empty", "DiagnosticCode")
        raw = self.message.encode("utf-8")
        if not raw:
            raise HostContractError("Empty", "DiagnosticMessage")
        if len(raw) > MAX_DIAGNOSTIC_MESSAGE_BYTES_V1:
            raise HostContractError("LimitExceeded", "DiagnosticMessage")
        if b"\0" in raw:
            raise HostContractError("DiagnosticContainsNul")

    def encode(self, e):
        e.u32(self.code)
        e.u8(self.severity)
        e.optional_digest(self.subject)
        e.text(self.message)


@dataclass(frozen=True)
class DispatchRequest:
    """dispatch.rs:96-268.  `identity` is the caller's commitment and is not part of the preimage."""
    identity: bytes
    context: OperationContext
    load_result: LoadedResult
    entry_point_identity: bytes
    dispatch_contract_identity: bytes
    argument_set_identity: bytes
    bindings: Tuple[ResourceBinding, ...] = ()
    dependencies: Tuple[DispatchDependency, ...] = ()
    kind: Optional[PersistentTask] = None          # None = one finite kernel dispatch

    def __post_init__(self):
        if len(self.bindings) > MAX_DISPATCH_BINDINGS_V1:
            raise HostContractError("TooManyItems", "DispatchBindings")
        for expected, b in enumerate(self.bindings):
            if b.ordinal != expected:
                raise HostContractError("NonCanonicalOrder", "DispatchBindings")
        deps = list(self.dependencies)
        _strictly_ordered(deps, MAX_DISPATCH_DEPENDENCIES_V1, "DispatchDependencies")
        if any(a.completion_signal_identity == b.completion_signal_identity for a, b in zip(deps, deps[1:])):
            raise HostContractError("Duplicate", "DispatchDependencies")
        if self.kind is not None and self.kind.service_epoch == 0:
            raise HostContractError("Empty", "ServiceEpoch")
        if self.load_result.load_generation == 0:
            raise HostContractError("InvalidOutcome")

    def encode_identity_preimage(self):
        e = Encoder(DOMAINS["DispatchRequestId"])
        self.context.encode(e)
        e.digest(self.load_result.identity)
        e.digest(self.load_result.loaded_object_identity)
        e.u64(self.load_result.load_generation)
        e.digest(self.entry_point_identity)
        e.digest(self.dispatch_contract_identity)
        e.digest(self.argument_set_identity)
        if self.kind is None:
            e.u8(1)
        else:
            e.u8(2)
            e.digest(self.kind.service_instance_identity)
            e.digest(self.kind.task_schema_identity)
            e.u32(self.kind.task_tag)
            e.u64(self.kind.service_epoch)
        e.u16(len(self.bindings))
        for b in self.bindings:
            b.encode(e)
        e.u16(len(self.dependencies))
        for d in self.dependencies:
            d.encode(e)
        return e.finish()


OUTCOME_SUBMITTED, OUTCOME_REJECTED, OUTCOME_FAILED = 1, 2, 3


@dataclass(frozen=True)
class DispatchResult:
    """dispatch.rs:270-368: the result of one dispatch request, bound to that request."""
    identity: bytes
    request: DispatchRequest
    outcome: int
    submission_identity: Optional[bytes] = None
    completion_signal_identity: Optional[bytes] = None
    diagnostics: Tuple[Diagnostic, ...] = field(default_factory=tuple)

    def __post_init__(self):
        if len(self.diagnostics) > MAX_DIAGNOSTICS_V1:
            raise HostContractError("TooManyItems", "Diagnostics")
        has_error = any(d.severity == SEVERITY_ERROR for d in self.diagnostics)
        if self.outcome in (OUTCOME_REJECTED, OUTCOME_FAILED) and not has_error:
            raise HostContractError("MissingFailureDiagnostic")
        if self.outcome == OUTCOME_SUBMITTED:
            if has_error or self.submission_identity is None or self.completion_signal_identity is None:
                raise HostContractError("InvalidOutcome")
        elif self.outcome not in (OUTCOME_REJECTED, OUTCOME_FAILED):
            raise HostContractError("InvalidOutcome")

    def encode_identity_preimage(self):
        e = Encoder(DOMAINS["DispatchResultId"])
        e.digest(self.request.identity)
        e.digest(self.request.load_result.loaded_object_identity)
        e.u8(self.outcome)
        if self.outcome == OUTCOME_SUBMITTED:
            e.digest(self.submission_identity)
            e.digest(self.completion_signal_identity)
        e.u16(len(self.diagnostics))
        for d in self.diagnostics:
            d.encode(e)
        return e.finish()


# ------------------------------------------------------------------ compile, admit and load flows
RESULT_SUCCEEDED, RESULT_REJECTED, RESULT_FAILED = 1, 2, 3   # outcome tags shared by the three flows


def _check_result_diagnostics(outcome, diagnostics):
    """common.rs:638-657 plus the rule each result repeats: a success carries no error diagnostic."""
    if outcome not in (RESULT_SUCCEEDED, RESULT_REJECTED, RESULT_FAILED):
        raise HostContractError("InvalidOutcome")
    if len(diagnostics) > MAX_DIAGNOSTICS_V1:
        raise HostContractError("TooManyItems", "Diagnostics")
    has_error = any(d.severity == SEVERITY_ERROR for d in diagnostics)
    if outcome != RESULT_SUCCEEDED and not has_error:
        raise HostContractError("MissingFailureDiagnostic")
    return has_error


def _encode_diagnostics(e, diagnostics):
    e.u16(len(diagnostics))
    for d in diagnostics:
        d.encode(e)


@dataclass(frozen=True)
class PayloadDescriptor:
    """common.rs:347-400: identity, format and byte length of an opaque payload."""
    identity: bytes
    format_identity: bytes
    byte_len: int

    def __post_init__(self):
        if self.byte_len == 0:
            raise HostContractError("Empty", "PayloadBytes")
        if self.byte_len > MAX_PAYLOAD_BYTES_V1:
            raise HostContractError("LimitExceeded", "PayloadBytes")

    def encode(self, e):
        e.digest(self.identity)
        e.digest(self.format_identity)
        e.u64(self.byte_len)


@dataclass(frozen=True)
class CompileRequest:
    """compile.rs:22-131."""
    identity: bytes
    context: OperationContext
    input: PayloadDescriptor
    compiler_profile_identity: bytes
    target_profile_identity: bytes
    configuration_identity: bytes
    maximum_output_bytes: int

    def __post_init__(self):
        if self.maximum_output_bytes == 0:
            raise HostContractError("Empty", "CompileOutputBytes")
        if self.maximum_output_bytes > MAX_PAYLOAD_BYTES_V1:
            raise HostContractError("LimitExceeded", "CompileOutputBytes")

    def encode_identity_preimage(self):
        e = Encoder(DOMAINS["CompileRequestId"])
        self.context.encode(e)
        self.input.encode(e)
        e.digest(self.compiler_profile_identity)
        e.digest(self.target_profile_identity)
        e.digest(self.configuration_identity)
        e.u64(self.maximum_output_bytes)
        return e.finish()


@dataclass(frozen=True)
class CompileResult:
    """compile.rs:133-219: `candidate` is the compiled payload of a successful compile."""
    identity: bytes
    request: CompileRequest
    outcome: int
    candidate: Optional[PayloadDescriptor] = None
    diagnostics: Tuple[Diagnostic, ...] = field(default_factory=tuple)

    def __post_init__(self):
        has_error = _check_result_diagnostics(self.outcome, self.diagnostics)
        if self.outcome == RESULT_SUCCEEDED:
            if self.candidate is None:
                raise HostContractError("InvalidOutcome")
            if self.candidate.byte_len > self.request.maximum_output_bytes:
                raise HostContractError("LimitExceeded", "CompileOutputBytes")
            if has_error:
                raise HostContractError("InvalidOutcome")
        elif self.candidate is not None:
            raise HostContractError("InvalidOutcome")

    def encode_identity_preimage(self):
        e = Encoder(DOMAINS["CompileResultId"])
        e.digest(self.request.identity)
        e.u8(self.outcome)
        if self.outcome == RESULT_SUCCEEDED:
            self.candidate.encode(e)
        _encode_diagnostics(e, self.diagnostics)
        return e.finish()


@dataclass(frozen=True)
class AdmitRequest:
    """admit.rs:29-117: admission of exactly the candidate a successful compile produced."""
    identity: bytes
    context: OperationContext
    compile_result: CompileResult
    candidate: PayloadDescriptor
    policy_identity: bytes
    required_claims: Tuple[bytes, ...] = ()

    def __post_init__(self):
        _strictly_ordered([digest(c) for c in self.required_claims], MAX_ADMISSION_CLAIMS_V1, "AdmissionClaims")
        if self.compile_result.outcome != RESULT_SUCCEEDED:
            raise HostContractError("InvalidOutcome")
        if self.compile_result.candidate != self.candidate:
            raise HostContractError("Mismatch", "UpstreamObject")

    def encode_identity_preimage(self):
        e = Encoder(DOMAINS["AdmitRequestId"])
        self.context.encode(e)
        e.digest(self.compile_result.identity)
        self.candidate.encode(e)
        e.digest(self.policy_identity)
        e.u16(len(self.required_claims))
        for c in self.required_claims:
            e.digest(c)
        return e.finish()


@dataclass(frozen=True)
class AdmitResult:
    """admit.rs:119-219: `assessment_identity` is set exactly when the candidate was accepted."""
    identity: bytes
    request: AdmitRequest
    outcome: int
    assessment_identity: Optional[bytes] = None
    diagnostics: Tuple[Diagnostic, ...] = field(default_factory=tuple)

    def __post_init__(self):
        has_error = _check_result_diagnostics(self.outcome, self.diagnostics)
        if self.outcome == RESULT_SUCCEEDED and (has_error or self.assessment_identity is None):
            raise HostContractError("InvalidOutcome")
        if self.outcome != RESULT_SUCCEEDED and self.assessment_identity is not None:
            raise HostContractError("InvalidOutcome")

    @property
    def candidate_identity(self):
        return self.request.candidate.identity

    def encode_identity_preimage(self):
        e = Encoder(DOMAINS["AdmitResultId"])
        e.digest(self.request.identity)
        e.digest(self.candidate_identity)
        e.u8(self.outcome)
        if self.outcome == RESULT_SUCCEEDED:
            e.digest(self.assessment_identity)
        _encode_diagnostics(e, self.diagnostics)
        return e.finish()


@dataclass(frozen=True)
class LoadRequest:
    """load.rs:31-117: a load of the artifact an accepted admission names."""
    identity: bytes
    context: OperationContext
    admit_result: AdmitResult
    artifact_identity: bytes
    loader_profile_identity: bytes
    runtime_context_identity: bytes

    def __post_init__(self):
        if self.admit_result.candidate_identity != self.artifact_identity:
            raise HostContractError("Mismatch", "UpstreamObject")
        if self.admit_result.outcome != RESULT_SUCCEEDED:
            raise HostContractError("InvalidOutcome")

    def encode_identity_preimage(self):
        e = Encoder(DOMAINS["LoadRequestId"])
        self.context.encode(e)
        e.digest(self.admit_result.identity)
        e.digest(self.admit_result.assessment_identity)
        e.digest(self.artifact_identity)
        e.digest(self.loader_profile_identity)
        e.digest(self.runtime_context_identity)
        return e.finish()


@dataclass(frozen=True)
class LoadResult:
    """load.rs:119-239: a successful load names the loaded object and a non-zero generation."""
    identity: bytes
    request: LoadRequest
    outcome: int
    loaded_object_identity: Optional[bytes] = None
    load_generation: int = 0
    diagnostics: Tuple[Diagnostic, ...] = field(default_factory=tuple)

    def __post_init__(self):
        has_error = _check_result_diagnostics(self.outcome, self.diagnostics)
        if self.outcome == RESULT_SUCCEEDED:
            if self.loaded_object_identity is None:
                raise HostContractError("InvalidOutcome")
            if self.load_generation == 0:
                raise HostContractError("Empty", "LoadGeneration")
            if has_error:
                raise HostContractError("InvalidOutcome")
        elif self.loaded_object_identity is not None:
            raise HostContractError("InvalidOutcome")

    def loaded(self):
        """What a dispatch request binds to (dispatch.rs:113-131 accepts only a successful load)."""
        if self.outcome != RESULT_SUCCEEDED:
            raise HostContractError("InvalidOutcome")
        return LoadedResult(self.identity, self.loaded_object_identity, self.load_generation)

    def encode_identity_preimage(self):
        e = Encoder(DOMAINS["LoadResultId"])
        e.digest(self.request.identity)
        e.digest(self.request.artifact_identity)
        e.digest(self.request.runtime_context_identity)
        e.u8(self.outcome)
        if self.outcome == RESULT_SUCCEEDED:
            e.digest(self.loaded_object_identity)
            e.u64(self.load_generation)
        _encode_diagnostics(e, self.diagnostics)
        return e.finish()


# ------------------------------------------------------------------ wait flow (src/wait.rs)
WAIT_ANY, WAIT_ALL = 1, 2                                                              # wait.rs:20-27
COMPLETION_SUCCEEDED, COMPLETION_CANCELLED, COMPLETION_FAILED = 1, 2, 3                # wait.rs:30-39
WAIT_SATISFIED, WAIT_PENDING, WAIT_REJECTED, WAIT_FAILED = 1, 2, 3, 4                  # tags of wait.rs:309-320


@dataclass(frozen=True)
class CompletionObservation:
    """wait.rs:42-83: one terminal observation of a completion signal."""
    signal_identity: bytes
    record_identity: bytes
    status: int

    def __post_init__(self):
        if self.status not in (COMPLETION_SUCCEEDED, COMPLETION_CANCELLED, COMPLETION_FAILED):
            raise HostContractError("InvalidOutcome")

    def encode(self, e):
        e.digest(self.signal_identity)
        e.digest(self.record_identity)
        e.u8(self.status)


@dataclass(frozen=True)
class WaitRequest:
    """wait.rs:107-207: a wait over a non-empty, strictly ordered set of completion signals."""
    identity: bytes
    context: OperationContext
    mode: int
    targets: Tuple[bytes, ...]
    deadline_identity: Optional[bytes] = None

    def __post_init__(self):
        if self.mode not in (WAIT_ANY, WAIT_ALL):
            raise HostContractError("InvalidOutcome")
        if not self.targets:
            raise HostContractError("Empty", "WaitTargets")
        _strictly_ordered([digest(t) for t in self.targets], MAX_WAIT_TARGETS_V1, "WaitTargets")

    def validate_dispatch_results(self, dispatch_results):
        """wait.rs:170-194: exactly one submitted dispatch result per target, and nothing else."""
        if len(dispatch_results) != len(self.targets):
            raise HostContractError("MissingDispatchResult")
        for target in self.targets:
            matching = sum(1 for r in dispatch_results
                           if r.outcome == OUTCOME_SUBMITTED and r.completion_signal_identity == target)
            if matching != 1:
                raise HostContractError("MissingDispatchResult")

    def encode_identity_preimage(self):
        e = Encoder(DOMAINS["WaitRequestId"])
        self.context.encode(e)
        e.u8(self.mode)
        e.u16(len(self.targets))
        for t in self.targets:
            e.digest(t)
        e.optional_digest(self.deadline_identity)
        return e.finish()


@dataclass(frozen=True)
class WaitResult:
    """wait.rs:209-325: the result of one wait request; target membership and the truth of the
    Any / All predicate are checked against the request."""
    identity: bytes
    request: WaitRequest
    outcome: int
    observations: Tuple[CompletionObservation, ...] = ()
    diagnostics: Tuple[Diagnostic, ...] = field(default_factory=tuple)

    def __post_init__(self):
        if self.outcome not in (WAIT_SATISFIED, WAIT_PENDING, WAIT_REJECTED, WAIT_FAILED):
            raise HostContractError("InvalidOutcome")
        if len(self.diagnostics) > MAX_DIAGNOSTICS_V1:
            raise HostContractError("TooManyItems", "Diagnostics")
        has_error = any(d.severity == SEVERITY_ERROR for d in self.diagnostics)
        if self.outcome in (WAIT_REJECTED, WAIT_FAILED):
            if not has_error:
                raise HostContractError("MissingFailureDiagnostic")
            if self.observations:
                raise HostContractError("InvalidOutcome")   # the reference's Rejected / Failed carry none
            return
        obs = self.observations
        if len(obs) > MAX_WAIT_TARGETS_V1:
            raise HostContractError("TooManyItems", "WaitObservations")
        for a, b in zip(obs, obs[1:]):
            if a.signal_identity == b.signal_identity:
                raise HostContractError("Duplicate", "WaitObservations")
            if a.signal_identity > b.signal_identity:
                raise HostContractError("NonCanonicalOrder", "WaitObservations")
        targets = set(self.request.targets)
        if any(o.signal_identity not in targets for o in obs):
            raise HostContractError("UnknownWaitTarget")
        satisfied = len(obs) > 0 if self.request.mode == WAIT_ANY else len(obs) == len(self.request.targets)
        if satisfied != (self.outcome == WAIT_SATISFIED):
            raise HostContractError("InvalidWaitDisposition")
        if has_error:
            raise HostContractError("InvalidOutcome")

    def encode_identity_preimage(self):
        e = Encoder(DOMAINS["WaitResultId"])
        e.digest(self.request.identity)
        e.u8(self.request.mode)
        e.u8(self.outcome)
        if self.outcome in (WAIT_SATISFIED, WAIT_PENDING):
            e.u16(len(self.observations))
            for o in self.observations:
                o.encode(e)
        e.u16(len(self.diagnostics))
        for d in self.diagnostics:
            d.encode(e)
        return e.finish()


# ------------------------------------------------------------------ operation states and events
PHASE_REQUESTED, PHASE_PENDING, PHASE_ACTIVE = 1, 2, 3                                 # tags of state.rs:245-262
PHASE_SUCCEEDED, PHASE_REJECTED, PHASE_FAILED, PHASE_CANCELLED = 4, 5, 6, 7
_TERMINAL = (PHASE_SUCCEEDED, PHASE_REJECTED, PHASE_FAILED, PHASE_CANCELLED)
_WITH_RESULT = (PHASE_SUCCEEDED, PHASE_REJECTED, PHASE_FAILED)
_FLOW_NAMES = {FLOW_COMPILE: "compile", FLOW_ADMIT: "admit", FLOW_LOAD: "load", FLOW_DISPATCH: "dispatch", FLOW_WAIT: "wait"}


def _flow_domain(flow, kind):
    return b"fe2o3.host." + _FLOW_NAMES[flow].encode() + b"." + kind + b".v1"


def can_transition(current, nxt):
    """state.rs:213-243: phases only move forward, and nothing follows a terminal phase."""
    if current == PHASE_REQUESTED:
        return nxt in (PHASE_PENDING, PHASE_ACTIVE) + _TERMINAL
    if current == PHASE_PENDING:
        return nxt in (PHASE_ACTIVE,) + _TERMINAL
    if current == PHASE_ACTIVE:
        return nxt in _TERMINAL
    return False


@dataclass(frozen=True)
class Phase:
    """state.rs:14-53: `result` = (flow, result identity) for the three phases that carry one."""
    tag: int
    result: Optional[Tuple[int, bytes]] = None

    def __post_init__(self):
        if self.tag not in range(1, 8) or (self.tag in _WITH_RESULT) != (self.result is not None):
            raise HostContractError("InvalidOutcome")

    @property
    def is_terminal(self):
        return self.tag in _TERMINAL

    def encode(self, e):
        e.u8(self.tag)
        if self.result is not None:
            e.digest(self.result[1])


REQUESTED = Phase(PHASE_REQUESTED)


@dataclass(frozen=True)
class OperationState:
    """state.rs:55-211: one link of an operation's state chain.  Build with `initial` and `transition`;
    every identity is a (flow, digest) pair, as the reference's flow-tagged identity enums are."""
    identity: Tuple[int, bytes]
    scope_id: bytes
    operation_id: bytes
    request_identity: Tuple[int, bytes]
    revision: int
    predecessor_identity: Optional[Tuple[int, bytes]]
    phase: Phase

    @classmethod
    def initial(cls, identity, context, request_identity):
        if identity[0] != request_identity[0]:
            raise HostContractError("Mismatch", "Flow")
        return cls(identity, context.scope_id, context.operation_id, request_identity, 0, None, REQUESTED)

    def transition(self, identity, phase):
        if self.phase.is_terminal:
            raise HostContractError("TerminalStateTransition")
        if identity[0] != self.identity[0]:
            raise HostContractError("Mismatch", "Flow")
        if identity == self.identity:
            raise HostContractError("Duplicate", "StateIdentity")
        if phase.result is not None and phase.result[0] != self.request_identity[0]:
            raise HostContractError("Mismatch", "TerminalResult")
        if not can_transition(self.phase.tag, phase.tag):
            raise HostContractError("InvalidStateTransition")
        if self.revision + 1 >= 1 << 32:
            raise HostContractError("ArithmeticOverflow", "StateRevision")
        return OperationState(identity, self.scope_id, self.operation_id, self.request_identity, self.revision + 1,
                              self.identity, phase)

    def validate_terminal_result(self, result_identity, request_identity, result_class):
        """state.rs:160-177: the terminal phase names exactly this result (identity and class) of this request.
        result_class: RESULT_SUCCEEDED / RESULT_REJECTED / RESULT_FAILED."""
        if request_identity != self.request_identity:
            raise HostContractError("Mismatch", "RequestIdentity")
        klass = {PHASE_SUCCEEDED: RESULT_SUCCEEDED, PHASE_REJECTED: RESULT_REJECTED, PHASE_FAILED: RESULT_FAILED}.get(self.phase.tag)
        if self.phase.result != result_identity or klass != result_class:
            raise HostContractError("Mismatch", "TerminalResult")

    def _encode_body(self, e):
        e.digest(self.scope_id)
        e.digest(self.operation_id)
        e.u8(self.request_identity[0])
        e.digest(self.request_identity[1])
        e.u32(self.revision)
        e.optional_digest(None if self.predecessor_identity is None else self.predecessor_identity[1])

    def encode_identity_preimage(self):
        e = Encoder(_flow_domain(self.identity[0], b"state"))
        self._encode_body(e)
        self.phase.encode(e)
        return e.finish()


@dataclass(frozen=True)
class Event:
    """event.rs:19-95: the event that announces one state of the chain."""
    identity: Tuple[int, bytes]
    state: OperationState

    def __post_init__(self):
        if self.identity[0] != self.state.identity[0]:
            raise HostContractError("Mismatch", "Flow")

    def validate_state(self, state):
        if state != self.state:
            raise HostContractError("Mismatch", "StatePredecessor")

    def encode_identity_preimage(self):
        e = Encoder(_flow_domain(self.identity[0], b"event"))
        self.state._encode_body(e)
        e.digest(self.state.identity[1])
        self.state.phase.encode(e)
        return e.finish()


@dataclass(frozen=True)
class EventBatch:
    """event.rs:97-205: events of one scope in producer order; the events of each operation form an unbroken
    chain from its Requested state, while different operations may interleave freely."""
    scope_id: bytes
    events: Tuple[Event, ...]

    def __post_init__(self):
        if not self.events:
            raise HostContractError("Empty", "EventBatch")
        if len(self.events) > MAX_EVENT_BATCH_V1:
            raise HostContractError("TooManyItems", "EventBatch")
        for index, event in enumerate(self.events):
            cur, earlier = event.state, self.events[:index]
            if cur.scope_id != self.scope_id:
                raise HostContractError("Mismatch", "Scope")
            if any(x.identity == event.identity for x in earlier):
                raise HostContractError("Duplicate", "EventBatch")
            if any(x.state.identity == cur.identity for x in earlier):
                raise HostContractError("Duplicate", "StateIdentity")
            previous = next((x.state for x in reversed(earlier) if x.state.operation_id == cur.operation_id), None)
            if previous is None:
                if cur.revision != 0 or cur.predecessor_identity is not None or cur.phase != REQUESTED:
                    raise HostContractError("InvalidInitialState")
                continue
            if previous.request_identity != cur.request_identity:
                raise HostContractError("Mismatch", "RequestIdentity")
            if cur.revision != previous.revision + 1:
                raise HostContractError("Mismatch", "StateRevision")
            if cur.predecessor_identity != previous.identity:
                raise HostContractError("Mismatch", "StatePredecessor")
            if previous.phase.is_terminal:
                raise HostContractError("TerminalStateTransition")
            if not can_transition(previous.phase.tag, cur.phase.tag):
                raise HostContractError("InvalidStateTransition")


# ------------------------------------------------------------------ this library's launches
def commit(domain_name, *parts):
    """A commitment an integration may choose: SHA-256 over the identity's domain and the given parts.
    The reference leaves the digest operation to the integration (identity.rs:6-9)."""
    h = hashlib.sha256(DOMAINS[domain_name])
    for p in parts:
        h.update(len(p).to_bytes(8, "little"))
        h.update(p)
    return h.digest()


def dispatch_request_for(prepared, op_args, context, load_result, written=(), element_bytes=None):
    """The dispatch request that describes one prepared launch of this library: entry point = the kernel
    symbol, argument set = the packed argument bytes, one binding per non-empty slice argument in
    declaration order.  `written` names the slices the kernel writes; `element_bytes` maps a slice name to
    its element size (slice lengths are in elements; default 4 bytes)."""
    from ._lib import Slice
    bindings, ordinal = [], 0
    for name, ty in type(op_args)._fields_:
        if ty is not Slice:
            continue
        s = getattr(op_args, name)
        if s.len == 0:
            continue
        resource = commit("ResourceId", name.encode(), int(s.ptr).to_bytes(8, "little"))
        size = (element_bytes or {}).get(name, 4)
        bindings.append(ResourceBinding(ordinal, resource, ACCESS_WRITE if name in written else ACCESS_READ, 0, int(s.len) * size))
        ordinal += 1
    kernarg = prepared.kernarg
    req = DispatchRequest(
        identity=bytes(32), context=context, load_result=load_result,
        entry_point_identity=commit("EntryPointId", prepared.symbol.encode()),
        dispatch_contract_identity=commit("DispatchContractId", prepared.symbol.encode(), len(kernarg).to_bytes(8, "little")),
        argument_set_identity=commit("ArgumentSetId", kernarg), bindings=tuple(bindings))
    ident = hashlib.sha256(req.encode_identity_preimage()).digest()
    return DispatchRequest(ident, req.context, req.load_result, req.entry_point_identity, req.dispatch_contract_identity,
                           req.argument_set_identity, req.bindings, req.dependencies, req.kind)


def wait_request_for(dispatch_results, context, mode=WAIT_ALL, deadline_identity=None):
    """The wait request over the completion signals of the given submitted dispatch results (targets in
    canonical order), checked against those results; its identity is the SHA-256 of its preimage."""
    targets = tuple(sorted(r.completion_signal_identity for r in dispatch_results if r.outcome == OUTCOME_SUBMITTED))
    req = WaitRequest(bytes(32), context, mode, targets, deadline_identity)
    req.validate_dispatch_results(list(dispatch_results))
    ident = hashlib.sha256(req.encode_identity_preimage()).digest()
    return WaitRequest(ident, context, mode, targets, deadline_identity)
