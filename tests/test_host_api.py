"""Dispatch and wait records of the host API: canonical preimages and structural rejections.

The properties checked are those of crates/fe2o3-host-api/tests/hostile_invariants.rs
(:159-228 identity domains and preimages, :236-317 scalar bounds, :319-368 upstream substitution,
:539-668 interleaved state chains, :670-768 stale / skipped / terminal states, :771-884 wait predicates, :887-941 preimage bounds) plus byte-level layouts
written out from crates/fe2o3-host-api/src/canonical.rs:13-21 and src/dispatch.rs:234-268.
"""
import struct

import pytest

from fe2o3_b200 import host_api as ha


def d(byte):
    return bytes([byte]) * 32


def context(**kw):
    return ha.OperationContext(d(1), d(2), kw.pop("attempt", 1), kw.pop("parent", None), kw.pop("events", ()))


LOADED = ha.LoadedResult(d(3), d(4), 7)


def request(**kw):
    return ha.DispatchRequest(kw.pop("identity", d(9)), kw.pop("context", context()), kw.pop("load", LOADED), d(5), d(6), d(7),
                              kw.pop("bindings", ()), kw.pop("dependencies", ()), kw.pop("kind", None))


def test_identity_domains_are_unique_and_preimages_start_with_magic_and_domain():
    assert len(set(ha.DOMAINS.values())) == len(ha.DOMAINS)
    assert all(v.startswith(b"fe2o3.host.") and v.endswith(b".v1") for v in ha.DOMAINS.values())
    pre = request().encode_identity_preimage()
    dom = ha.DOMAINS["DispatchRequestId"]
    assert pre.startswith(b"F2HOSTP1" + struct.pack("<H", len(dom)) + dom + struct.pack("<H", 1))


def test_finite_dispatch_request_preimage_layout_byte_for_byte():
    b0 = ha.ResourceBinding(0, d(0x10), ha.ACCESS_READ, 16, 4096)
    b1 = ha.ResourceBinding(1, d(0x11), ha.ACCESS_WRITE, 0, 64)
    dep = ha.DispatchDependency(d(0x20), d(0x21))
    ctx = context(attempt=3, parent=d(8), events=((ha.FLOW_LOAD, d(0x30)), (ha.FLOW_DISPATCH, d(0x2f))))
    pre = request(context=ctx, bindings=(b0, b1), dependencies=(dep,)).encode_identity_preimage()
    dom = ha.DOMAINS["DispatchRequestId"]
    want = (b"F2HOSTP1" + struct.pack("<H", len(dom)) + dom + struct.pack("<H", 1)
            + d(1) + d(2) + struct.pack("<H", 3) + b"\x01" + d(8)                       # context
            + struct.pack("<H", 2) + b"\x03" + d(0x30) + b"\x04" + d(0x2f)                 # causal events
            + d(3) + d(4) + struct.pack("<Q", 7) + d(5) + d(6) + d(7) + b"\x01"          # load result, ids, finite
            + struct.pack("<H", 2)
            + struct.pack("<H", 0) + d(0x10) + b"\x01" + struct.pack("<QQ", 16, 4096)
            + struct.pack("<H", 1) + d(0x11) + b"\x02" + struct.pack("<QQ", 0, 64)
            + struct.pack("<H", 1) + d(0x20) + d(0x21))
    assert pre == want


def test_preimage_excludes_the_declared_identity_and_covers_every_field():
    first = request()
    assert first.encode_identity_preimage() == request(identity=d(0x77)).encode_identity_preimage()
    variants = [request(context=context(attempt=2)), request(load=ha.LoadedResult(d(3), d(4), 8)),
                request(bindings=(ha.ResourceBinding(0, d(1), ha.ACCESS_ATOMIC, 0, 1),)),
                request(dependencies=(ha.DispatchDependency(d(1), d(2)),)),
                request(kind=ha.PersistentTask(d(1), d(2), 5, 1))]
    pres = {v.encode_identity_preimage() for v in variants} | {first.encode_identity_preimage()}
    assert len(pres) == len(variants) + 1


def test_persistent_task_kind_is_encoded_after_tag_two():
    pre = request(kind=ha.PersistentTask(d(0x41), d(0x42), 0xdeadbeef, 9)).encode_identity_preimage()
    assert b"\x02" + d(0x41) + d(0x42) + struct.pack("<IQ", 0xdeadbeef, 9) + struct.pack("<HH", 0, 0) == pre[-(1 + 64 + 12 + 4):]


def test_structural_rejections():
    with pytest.raises(ha.HostContractError) as e:
        context(attempt=0)
    assert (e.value.kind, e.value.field) == ("Empty", "OperationAttempt")
    with pytest.raises(ha.HostContractError) as e:
        context(parent=d(2))
    assert (e.value.kind, e.value.field) == ("Mismatch", "ParentOperation")
    with pytest.raises(ha.HostContractError) as e:
        context(events=((ha.FLOW_WAIT, d(1)), (ha.FLOW_LOAD, d(1))))
    assert e.value.kind == "NonCanonicalOrder"
    with pytest.raises(ha.HostContractError) as e:
        context(events=((ha.FLOW_LOAD, d(1)), (ha.FLOW_LOAD, d(1))))
    assert e.value.kind == "Duplicate"
    with pytest.raises(ha.HostContractError) as e:
        ha.ResourceBinding(0, d(1), ha.ACCESS_READ, 0, 0)
    assert (e.value.kind, e.value.field) == ("Empty", "ResourceRange")
    with pytest.raises(ha.HostContractError) as e:
        ha.ResourceBinding(0, d(1), ha.ACCESS_READ, (1 << 64) - 8, 8)
    assert e.value.kind == "ArithmeticOverflow"
    with pytest.raises(ha.HostContractError) as e:      # ordinals must be 0, 1, 2, ...
        request(bindings=(ha.ResourceBinding(1, d(1), ha.ACCESS_READ, 0, 1),))
    assert (e.value.kind, e.value.field) == ("NonCanonicalOrder", "DispatchBindings")
    with pytest.raises(ha.HostContractError) as e:
        request(bindings=tuple(ha.ResourceBinding(i, d(1), ha.ACCESS_READ, 0, 1) for i in range(129)))
    assert e.value.kind == "TooManyItems"
    with pytest.raises(ha.HostContractError) as e:      # two dependencies on one completion signal
        request(dependencies=(ha.DispatchDependency(d(1), d(2)), ha.DispatchDependency(d(1), d(3))))
    assert (e.value.kind, e.value.field) == ("Duplicate", "DispatchDependencies")
    with pytest.raises(ha.HostContractError) as e:
        request(dependencies=(ha.DispatchDependency(d(2), d(2)), ha.DispatchDependency(d(1), d(3))))
    assert e.value.kind == "NonCanonicalOrder"
    with pytest.raises(ha.HostContractError) as e:
        request(kind=ha.PersistentTask(d(1), d(2), 1, 0))
    assert (e.value.kind, e.value.field) == ("Empty", "ServiceEpoch")


def test_dispatch_result_outcomes_and_diagnostics():
    req = request()
    ok = ha.DispatchResult(d(0x50), req, ha.OUTCOME_SUBMITTED, d(0x51), d(0x52),
                           (ha.Diagnostic(7, ha.SEVERITY_NOTE, "queued", subject=d(0x53)),))
    dom = ha.DOMAINS["DispatchResultId"]
    want = (b"F2HOSTP1" + struct.pack("<H", len(dom)) + dom + struct.pack("<H", 1) + d(9) + d(4) + b"\x01" + d(0x51) + d(0x52)
            + struct.pack("<H", 1) + struct.pack("<I", 7) + b"\x01" + b"\x01" + d(0x53) + struct.pack("<H", 6) + b"queued")
    assert ok.encode_identity_preimage() == want
    failed = ha.DispatchResult(d(0x50), req, ha.OUTCOME_FAILED, diagnostics=(ha.Diagnostic(1, ha.SEVERITY_ERROR, "no device"),))
    assert failed.encode_identity_preimage().endswith(b"\x03" + struct.pack("<H", 1) + struct.pack("<I", 1) + b"\x03\x00"
                                                      + struct.pack("<H", 9) + b"no device")
    with pytest.raises(ha.HostContractError) as e:      # a failure needs an error diagnostic
        ha.DispatchResult(d(0x50), req, ha.OUTCOME_REJECTED)
    assert e.value.kind == "MissingFailureDiagnostic"
    with pytest.raises(ha.HostContractError) as e:      # a submission may not carry an error diagnostic
        ha.DispatchResult(d(0x50), req, ha.OUTCOME_SUBMITTED, d(1), d(2), (ha.Diagnostic(1, ha.SEVERITY_ERROR, "x"),))
    assert e.value.kind == "InvalidOutcome"
    for bad, kind in (("", "Empty"), ("a\0b", "DiagnosticContainsNul"), ("x" * 1025, "LimitExceeded")):
        with pytest.raises(ha.HostContractError) as e:
            ha.Diagnostic(1, ha.SEVERITY_NOTE, bad)
        assert e.value.kind == kind
    with pytest.raises(ha.HostContractError):
        ha.Diagnostic(0, ha.SEVERITY_NOTE, "zero code")


def test_maximum_valid_records_have_bounded_identity_preimages():
    events = tuple((ha.FLOW_DISPATCH, bytes([i]) * 32) for i in range(64))
    bindings = tuple(ha.ResourceBinding(i, d(1), ha.ACCESS_READ_WRITE, 0, 1) for i in range(128))
    deps = tuple(ha.DispatchDependency(bytes([i]) * 32, d(0)) for i in range(128))
    req = request(context=context(events=events), bindings=bindings, dependencies=deps,
                  kind=ha.PersistentTask(d(1), d(2), 3, 4))
    assert len(req.encode_identity_preimage()) <= ha.MAX_IDENTITY_PREIMAGE_BYTES_V1
    diags = tuple(ha.Diagnostic(1 + i, ha.SEVERITY_ERROR, "m" * 1024, subject=d(1)) for i in range(64))
    res = ha.DispatchResult(d(1), req, ha.OUTCOME_FAILED, diagnostics=diags)
    assert len(res.encode_identity_preimage()) <= ha.MAX_IDENTITY_PREIMAGE_BYTES_V1


# ---------------------------------------------------------------------------- wait flow
def wait_request(mode=None, targets=(d(0x40), d(0x41)), **kw):
    return ha.WaitRequest(kw.pop("identity", d(0x50)), kw.pop("context", context()),
                          ha.WAIT_ALL if mode is None else mode, tuple(targets), kw.pop("deadline", None))


def observed(sig, status=None):
    return ha.CompletionObservation(sig, d(0x60), ha.COMPLETION_SUCCEEDED if status is None else status)


def rejected(kind, field=None):
    return pytest.raises(ha.HostContractError, match=kind if field is None else f"{kind}\\({field}\\)")


def test_wait_request_rejects_empty_duplicate_unordered_and_oversized_target_sets():
    with rejected("Empty", "WaitTargets"):
        wait_request(ha.WAIT_ANY, targets=())
    with rejected("Duplicate", "WaitTargets"):
        wait_request(targets=(d(0x40), d(0x40)))
    with rejected("NonCanonicalOrder", "WaitTargets"):
        wait_request(targets=(d(0x41), d(0x40)))
    many = tuple((20_000 + i).to_bytes(32, "big") for i in range(ha.MAX_WAIT_TARGETS_V1 + 1))
    with rejected("TooManyItems", "WaitTargets"):
        wait_request(targets=many)
    assert len(wait_request(targets=many[:-1]).targets) == ha.MAX_WAIT_TARGETS_V1


def test_wait_result_checks_membership_order_and_the_predicate():
    a, b = d(0x40), d(0x41)
    any_req, all_req = wait_request(ha.WAIT_ANY), wait_request(ha.WAIT_ALL)
    with rejected("InvalidWaitDisposition"):      # Any is not satisfied by nothing
        ha.WaitResult(d(0x70), any_req, ha.WAIT_SATISFIED, ())
    with rejected("InvalidWaitDisposition"):      # Any with one observation is not pending
        ha.WaitResult(d(0x70), any_req, ha.WAIT_PENDING, (observed(a),))
    with rejected("UnknownWaitTarget"):
        ha.WaitResult(d(0x70), any_req, ha.WAIT_SATISFIED, (observed(d(0x99)),))
    with rejected("Duplicate", "WaitObservations"):
        ha.WaitResult(d(0x70), any_req, ha.WAIT_SATISFIED, (observed(a), observed(a)))
    with rejected("NonCanonicalOrder", "WaitObservations"):
        ha.WaitResult(d(0x70), all_req, ha.WAIT_SATISFIED, (observed(b), observed(a)))
    with rejected("InvalidWaitDisposition"):      # All needs every target
        ha.WaitResult(d(0x70), all_req, ha.WAIT_SATISFIED, (observed(a),))
    assert ha.WaitResult(d(0x70), all_req, ha.WAIT_PENDING, (observed(a),)).outcome == ha.WAIT_PENDING
    assert ha.WaitResult(d(0x70), any_req, ha.WAIT_PENDING, ()).observations == ()
    done = ha.WaitResult(d(0x70), all_req, ha.WAIT_SATISFIED, (observed(a), observed(b, ha.COMPLETION_FAILED)))
    assert len(done.observations) == 2
    err = ha.Diagnostic(7, ha.SEVERITY_ERROR, "device lost")
    with rejected("InvalidOutcome"):              # a successful wait carries no error diagnostic
        ha.WaitResult(d(0x70), any_req, ha.WAIT_SATISFIED, (observed(a),), (err,))
    with rejected("MissingFailureDiagnostic"):
        ha.WaitResult(d(0x70), any_req, ha.WAIT_FAILED)
    with rejected("MissingFailureDiagnostic"):
        ha.WaitResult(d(0x70), any_req, ha.WAIT_REJECTED, (), (ha.Diagnostic(7, ha.SEVERITY_WARNING, "slow"),))
    assert ha.WaitResult(d(0x70), any_req, ha.WAIT_FAILED, (), (err,)).diagnostics == (err,)


def test_wait_preimage_layouts_byte_for_byte():
    req = wait_request(ha.WAIT_ANY, context=context(attempt=2), deadline=d(0x55))
    dom = ha.DOMAINS["WaitRequestId"]
    head = b"F2HOSTP1" + struct.pack("<H", len(dom)) + dom + struct.pack("<H", 1)
    want = (head + d(1) + d(2) + struct.pack("<H", 2) + b"\x00" + struct.pack("<H", 0)    # context, no parent, no events
            + b"\x01" + struct.pack("<H", 2) + d(0x40) + d(0x41) + b"\x01" + d(0x55))
    assert req.encode_identity_preimage() == want
    assert wait_request(ha.WAIT_ANY, context=context(attempt=2)).encode_identity_preimage() == want[:-33] + b"\x00"
    assert req.encode_identity_preimage() == wait_request(ha.WAIT_ANY, context=context(attempt=2), deadline=d(0x55),
                                                          identity=d(0x51)).encode_identity_preimage()
    warn = ha.Diagnostic(3, ha.SEVERITY_NOTE, "ok", d(0x66))
    res = ha.WaitResult(d(0x70), req, ha.WAIT_SATISFIED, (observed(d(0x41), ha.COMPLETION_CANCELLED),), (warn,))
    dom = ha.DOMAINS["WaitResultId"]
    head = b"F2HOSTP1" + struct.pack("<H", len(dom)) + dom + struct.pack("<H", 1)
    want = (head + d(0x50) + b"\x01" + b"\x01" + struct.pack("<H", 1) + d(0x41) + d(0x60) + b"\x02"
            + struct.pack("<H", 1) + struct.pack("<I", 3) + b"\x01" + b"\x01" + d(0x66) + struct.pack("<H", 2) + b"ok")
    assert res.encode_identity_preimage() == want
    err = ha.Diagnostic(9, ha.SEVERITY_ERROR, "no")
    failed = ha.WaitResult(d(0x70), req, ha.WAIT_FAILED, (), (err,)).encode_identity_preimage()
    assert failed == (head + d(0x50) + b"\x01" + b"\x04" + struct.pack("<H", 1) + struct.pack("<I", 9) + b"\x03" + b"\x00"
                      + struct.pack("<H", 2) + b"no")


def test_wait_request_must_be_backed_by_exactly_its_submitted_dispatch_results():
    r1 = ha.DispatchResult(d(0x80), request(identity=d(0x0a)), ha.OUTCOME_SUBMITTED, d(0x81), d(0x41))
    r2 = ha.DispatchResult(d(0x82), request(identity=d(0x0b)), ha.OUTCOME_SUBMITTED, d(0x83), d(0x40))
    failed = ha.DispatchResult(d(0x84), request(identity=d(0x0c)), ha.OUTCOME_FAILED,
                               diagnostics=(ha.Diagnostic(1, ha.SEVERITY_ERROR, "launch failed"),))
    req = ha.wait_request_for([r1, r2], context())
    assert req.targets == (d(0x40), d(0x41)) and req.mode == ha.WAIT_ALL
    import hashlib
    assert req.identity == hashlib.sha256(req.encode_identity_preimage()).digest()
    req.validate_dispatch_results([r2, r1])
    for bad in ([r1], [r1, r1], [r1, failed], [r1, r2, failed]):
        with rejected("MissingDispatchResult"):
            req.validate_dispatch_results(bad)


# ---------------------------------------------------------------------------- compile -> admit -> load
def payload(byte, n):
    return ha.PayloadDescriptor(d(byte), d(byte + 1), n)


def compile_success(max_out=8192):
    creq = ha.CompileRequest(d(0xa0), context(), payload(0xa1, 2048), d(0xa3), d(0xa4), d(0xa5), max_out)
    cand = payload(0xa7, 4096)
    return creq, ha.CompileResult(d(0xa6), creq, ha.RESULT_SUCCEEDED, cand), cand


def accepted_load(generation=7):
    _, cres, cand = compile_success()
    areq = ha.AdmitRequest(d(0xb0), context(), cres, cand, d(0xb1), (d(0xb2),))
    ares = ha.AdmitResult(d(0xb3), areq, ha.RESULT_SUCCEEDED, d(0xb4))
    lreq = ha.LoadRequest(d(0xb5), context(), ares, cand.identity, d(0xb6), d(0xb7))
    return ha.LoadResult(d(0xb8), lreq, ha.RESULT_SUCCEEDED, d(0xb9), generation)


ERR = ha.Diagnostic(1, ha.SEVERITY_ERROR, "error")


def test_scalar_bounds_fail_closed():
    with rejected("Empty", "PayloadBytes"):
        payload(1, 0)
    with rejected("LimitExceeded", "PayloadBytes"):
        payload(1, ha.MAX_PAYLOAD_BYTES_V1 + 1)
    with rejected("Empty", "CompileOutputBytes"):
        compile_success(0)
    with rejected("LimitExceeded", "CompileOutputBytes"):
        compile_success(ha.MAX_PAYLOAD_BYTES_V1 + 1)
    with rejected("LimitExceeded", "CompileOutputBytes"):      # the candidate is larger than the request allows
        compile_success(4095)
    creq, _, _ = compile_success()
    with rejected("MissingFailureDiagnostic"):
        ha.CompileResult(d(0xc0), creq, ha.RESULT_FAILED)
    with rejected("InvalidOutcome"):                             # a candidate with an error diagnostic
        ha.CompileResult(d(0xc1), creq, ha.RESULT_SUCCEEDED, payload(0xc2, 32), (ERR,))
    assert ha.CompileResult(d(0xc3), creq, ha.RESULT_REJECTED, None, (ERR,)).candidate is None


def test_upstream_substitution_and_noncanonical_claims_are_rejected():
    creq, cres, cand = compile_success()
    with rejected("Mismatch", "UpstreamObject"):                 # another payload of the same size
        ha.AdmitRequest(d(0xb0), context(), cres, payload(0x99, cand.byte_len), d(0xb1))
    failed_compile = ha.CompileResult(d(0xc3), creq, ha.RESULT_FAILED, None, (ERR,))
    with rejected("InvalidOutcome"):
        ha.AdmitRequest(d(0xb0), context(), failed_compile, cand, d(0xb1))
    with rejected("NonCanonicalOrder", "AdmissionClaims"):
        ha.AdmitRequest(d(0xb0), context(), cres, cand, d(0xb1), (d(2), d(1)))
    with rejected("Duplicate", "AdmissionClaims"):
        ha.AdmitRequest(d(0xb0), context(), cres, cand, d(0xb1), (d(1), d(1)))
    areq = ha.AdmitRequest(d(0xb0), context(), cres, cand, d(0xb1))
    with rejected("InvalidOutcome"):                             # accepted without an assessment
        ha.AdmitResult(d(0xb3), areq, ha.RESULT_SUCCEEDED)
    rejected_admit = ha.AdmitResult(d(0xb3), areq, ha.RESULT_REJECTED, None, (ERR,))
    with rejected("InvalidOutcome"):                             # a load needs an accepted admission
        ha.LoadRequest(d(0xb5), context(), rejected_admit, cand.identity, d(0xb6), d(0xb7))
    accepted = ha.AdmitResult(d(0xb3), areq, ha.RESULT_SUCCEEDED, d(0xb4))
    with rejected("Mismatch", "UpstreamObject"):                 # a load of some other artifact
        ha.LoadRequest(d(0xb5), context(), accepted, d(0x98), d(0xb6), d(0xb7))
    lreq = ha.LoadRequest(d(0xb5), context(), accepted, cand.identity, d(0xb6), d(0xb7))
    with rejected("Empty", "LoadGeneration"):
        ha.LoadResult(d(0xb8), lreq, ha.RESULT_SUCCEEDED, d(0xb9), 0)
    failed_load = ha.LoadResult(d(0xb8), lreq, ha.RESULT_FAILED, None, 0, (ERR,))
    with rejected("InvalidOutcome"):                             # a dispatch cannot bind to a failed load
        failed_load.loaded()


def test_flow_chain_feeds_a_dispatch_and_preimages_follow_the_reference_layouts():
    load = accepted_load()
    req = request(load=load.loaded())
    assert req.load_result == ha.LoadedResult(d(0xb8), d(0xb9), 7)
    ctx = d(1) + d(2) + struct.pack("<H", 1) + b"\x00" + struct.pack("<H", 0)

    def head(name):
        dom = ha.DOMAINS[name]
        return b"F2HOSTP1" + struct.pack("<H", len(dom)) + dom + struct.pack("<H", 1)

    creq, cres, cand = compile_success()
    assert creq.encode_identity_preimage() == (head("CompileRequestId") + ctx + d(0xa1) + d(0xa2) + struct.pack("<Q", 2048)
                                               + d(0xa3) + d(0xa4) + d(0xa5) + struct.pack("<Q", 8192))
    assert cres.encode_identity_preimage() == (head("CompileResultId") + d(0xa0) + b"\x01" + d(0xa7) + d(0xa8)
                                               + struct.pack("<Q", 4096) + struct.pack("<H", 0))
    lreq = load.request
    areq = lreq.admit_result.request
    assert areq.encode_identity_preimage() == (head("AdmitRequestId") + ctx + d(0xa6) + d(0xa7) + d(0xa8) + struct.pack("<Q", 4096)
                                               + d(0xb1) + struct.pack("<H", 1) + d(0xb2))
    assert lreq.admit_result.encode_identity_preimage() == (head("AdmitResultId") + d(0xb0) + d(0xa7) + b"\x01" + d(0xb4)
                                                            + struct.pack("<H", 0))
    assert lreq.encode_identity_preimage() == head("LoadRequestId") + ctx + d(0xb3) + d(0xb4) + d(0xa7) + d(0xb6) + d(0xb7)
    assert load.encode_identity_preimage() == (head("LoadResultId") + d(0xb5) + d(0xa7) + d(0xb7) + b"\x01" + d(0xb9)
                                               + struct.pack("<Q", 7) + struct.pack("<H", 0))
    failed = ha.LoadResult(d(0xb8), lreq, ha.RESULT_REJECTED, None, 0, (ERR,))
    assert failed.encode_identity_preimage() == (head("LoadResultId") + d(0xb5) + d(0xa7) + d(0xb7) + b"\x02" + struct.pack("<H", 1)
                                                 + struct.pack("<I", 1) + b"\x03" + b"\x00" + struct.pack("<H", 5) + b"error")


# ---------------------------------------------------------------------------- state chains and events
D = ha.FLOW_DISPATCH


def dispatch_pair(op_byte, ident_byte):
    ctx = ha.OperationContext(d(1), d(op_byte), 1)
    req = request(identity=d(ident_byte), context=ctx)
    return req, ha.DispatchResult(d(ident_byte + 1), req, ha.OUTCOME_SUBMITTED, d(ident_byte + 2), d(ident_byte + 3))


def test_parallel_dispatches_have_independent_interleavable_state_chains():
    req_a, res_a = dispatch_pair(0x0a, 0x10)
    req_b, res_b = dispatch_pair(0x0b, 0x20)
    a0 = ha.OperationState.initial((D, d(0x30)), req_a.context, (D, req_a.identity))
    a1 = a0.transition((D, d(0x31)), ha.Phase(ha.PHASE_PENDING))
    a2 = a1.transition((D, d(0x32)), ha.Phase(ha.PHASE_SUCCEEDED, (D, res_a.identity)))
    a2.validate_terminal_result((D, res_a.identity), (D, req_a.identity), ha.RESULT_SUCCEEDED)
    b0 = ha.OperationState.initial((D, d(0x40)), req_b.context, (D, req_b.identity))
    b1 = b0.transition((D, d(0x41)), ha.Phase(ha.PHASE_ACTIVE))
    b2 = b1.transition((D, d(0x42)), ha.Phase(ha.PHASE_SUCCEEDED, (D, res_b.identity)))
    b2.validate_terminal_result((D, res_b.identity), (D, req_b.identity), ha.RESULT_SUCCEEDED)
    assert (a2.revision, a2.predecessor_identity, b2.revision) == (2, a1.identity, 2)
    with rejected("Mismatch", "RequestIdentity"):
        a2.validate_terminal_result((D, res_b.identity), (D, req_b.identity), ha.RESULT_SUCCEEDED)
    with rejected("Mismatch", "TerminalResult"):      # the right request, another operation's result
        a2.validate_terminal_result((D, res_b.identity), (D, req_a.identity), ha.RESULT_SUCCEEDED)
    with rejected("Mismatch", "TerminalResult"):      # the right result under the wrong class
        a2.validate_terminal_result((D, res_a.identity), (D, req_a.identity), ha.RESULT_FAILED)
    ev = [ha.Event((D, st.identity[1]), st) for st in (a0, b0, b1, a1, b2, a2)]   # interleaved in producer order
    assert len(ha.EventBatch(d(1), tuple(ev)).events) == 6
    with rejected("Mismatch", "StateRevision"):       # b's chain with a link left out
        ha.EventBatch(d(1), (ev[0], ev[1], ev[4]))
    fork = a0.transition((D, d(0x33)), ha.Phase(ha.PHASE_ACTIVE))   # another successor of a0: a2 does not follow it
    with rejected("Mismatch", "StatePredecessor"):
        ha.EventBatch(d(1), (ev[0], ha.Event((D, d(0x33)), fork), ev[5]))
    with rejected("Mismatch", "Scope"):
        ha.EventBatch(d(2), tuple(ev))


def test_state_and_event_chains_reject_cross_flow_stale_skipped_and_terminal_use():
    req, res = dispatch_pair(0x0a, 0x10)
    with rejected("Mismatch", "Flow"):
        ha.OperationState.initial((ha.FLOW_LOAD, d(0x30)), req.context, (D, req.identity))
    s0 = ha.OperationState.initial((D, d(0x31)), req.context, (D, req.identity))
    with rejected("Mismatch", "TerminalResult"):      # a load result cannot end a dispatch
        s0.transition((D, d(0x32)), ha.Phase(ha.PHASE_SUCCEEDED, (ha.FLOW_LOAD, d(0x33))))
    with rejected("Mismatch", "Flow"):
        s0.transition((ha.FLOW_WAIT, d(0x32)), ha.Phase(ha.PHASE_PENDING))
    s1 = s0.transition((D, d(0x34)), ha.Phase(ha.PHASE_PENDING))
    with rejected("Duplicate", "StateIdentity"):
        s1.transition(s1.identity, ha.Phase(ha.PHASE_ACTIVE))
    with rejected("InvalidStateTransition"):          # phases do not move backwards
        s1.transition((D, d(0x35)), ha.REQUESTED)
    s2 = s1.transition((D, d(0x35)), ha.Phase(ha.PHASE_SUCCEEDED, (D, res.identity)))
    with rejected("TerminalStateTransition"):
        s2.transition((D, d(0x36)), ha.Phase(ha.PHASE_CANCELLED))
    with rejected("InvalidOutcome"):                  # a terminal result phase needs its result, the others take none
        ha.Phase(ha.PHASE_FAILED)
    e0, e1, e2 = (ha.Event((D, st.identity[1]), st) for st in (s0, s1, s2))
    with rejected("Mismatch", "Flow"):
        ha.Event((ha.FLOW_WAIT, d(0x31)), s0)
    with rejected("Mismatch", "StatePredecessor"):
        e0.validate_state(s1)
    e0.validate_state(s0)
    with rejected("Mismatch", "StateRevision"):       # a skipped link
        ha.EventBatch(d(1), (e0, e2))
    with rejected("Duplicate", "EventBatch"):
        ha.EventBatch(d(1), (e0, e0))
    with rejected("Duplicate", "StateIdentity"):
        ha.EventBatch(d(1), (e0, ha.Event((D, d(0x37)), s0)))
    with rejected("InvalidInitialState"):             # a chain that does not start at Requested
        ha.EventBatch(d(1), (e1, e2))
    with rejected("Empty", "EventBatch"):
        ha.EventBatch(d(1), ())
    assert len(ha.EventBatch(d(1), (e0, e1, e2)).events) == 3


def test_state_and_event_preimage_layouts():
    req, res = dispatch_pair(0x0a, 0x10)
    s0 = ha.OperationState.initial((D, d(0x31)), req.context, (D, req.identity))
    s1 = s0.transition((D, d(0x34)), ha.Phase(ha.PHASE_FAILED, (D, res.identity)))

    def head(dom):
        return b"F2HOSTP1" + struct.pack("<H", len(dom)) + dom + struct.pack("<H", 1)

    body0 = d(1) + d(0x0a) + b"\x04" + d(0x10) + struct.pack("<I", 0) + b"\x00"
    body1 = d(1) + d(0x0a) + b"\x04" + d(0x10) + struct.pack("<I", 1) + b"\x01" + d(0x31)
    assert s0.encode_identity_preimage() == head(b"fe2o3.host.dispatch.state.v1") + body0 + b"\x01"
    assert s1.encode_identity_preimage() == head(b"fe2o3.host.dispatch.state.v1") + body1 + b"\x06" + d(0x11)
    assert ha.Event((D, d(0x50)), s1).encode_identity_preimage() == (head(ha.DOMAINS["DispatchEventId"]) + body1 + d(0x34)
                                                                     + b"\x06" + d(0x11))
    w = ha.OperationState.initial((ha.FLOW_WAIT, d(0x60)), req.context, (ha.FLOW_WAIT, d(0x61)))
    assert w.encode_identity_preimage().startswith(head(b"fe2o3.host.wait.state.v1") + d(1) + d(0x0a) + b"\x05" + d(0x61))
