"""Table tests of the pure quorum rules (C++: csrc/control/quorum.cc).

Scenarios follow the reference's unit tests in src/lighthouse.rs:584-1037 and
src/manager.rs:720-850.
"""

import pytest

from torchft_b200 import _control as C


def member(rid, step=1, shrink_only=False, addr=None):
    return {
        "replica_id": rid,
        "address": addr or f"addr_{rid}",
        "store_address": f"store_{rid}",
        "step": step,
        "world_size": 1,
        "shrink_only": shrink_only,
    }


def part(rid, joined, **kw):
    return {"joined": joined, "member": member(rid, **kw)}


def test_join_timeout_waits_for_stragglers():
    now = 100.0
    state = {"participants": {}, "heartbeats": {}, "prev_quorum": None}
    members, reason = C.quorum_compute(now, state, min_replicas=1, join_timeout_ms=60000)
    assert members is None
    assert "New quorum not ready, only have 0 participants, need min_replicas 1" in reason

    state["participants"]["a"] = part("a", now)
    state["heartbeats"]["a"] = now
    members, reason = C.quorum_compute(now, state, min_replicas=1, join_timeout_ms=60000)
    assert members is not None and [m["replica_id"] for m in members] == ["a"]
    assert "Valid quorum found" in reason

    # c heartbeats but has not asked yet: wait for it until the join timeout passes
    state["participants"]["b"] = part("b", now)
    state["heartbeats"]["b"] = now
    state["heartbeats"]["c"] = now
    members, reason = C.quorum_compute(now, state, min_replicas=1, join_timeout_ms=60000)
    assert members is None
    assert "Valid quorum with 2 participants, waiting for 1 healthy but not participating stragglers due to join timeout" in reason

    members, reason = C.quorum_compute(now + 61.0, state, min_replicas=1, join_timeout_ms=60000, heartbeat_timeout_ms=10**9)
    assert members is not None and len(members) == 2
    assert "Valid quorum found" in reason


def test_heartbeat_expiry_drops_participant():
    now = 100.0
    state = {
        "participants": {"a": part("a", now), "b": part("b", now)},
        "heartbeats": {"a": now, "b": now - 10.0},  # b stopped 10 s ago (timeout 5 s)
        "prev_quorum": None,
    }
    members, reason = C.quorum_compute(now, state, min_replicas=1, join_timeout_ms=0)
    assert [m["replica_id"] for m in members] == ["a"]
    assert "[1/2 participants healthy][1 heartbeating]" in reason


def test_min_replicas():
    now = 5.0
    state = {"participants": {"a": part("a", now)}, "heartbeats": {"a": now}, "prev_quorum": None}
    members, reason = C.quorum_compute(now, state, min_replicas=2, join_timeout_ms=0)
    assert members is None
    assert "New quorum not ready, only have 1 participants, need min_replicas 2" in reason


def test_fast_quorum_and_expansion():
    now = 50.0
    prev = {"quorum_id": 1, "participants": [member("a"), member("b")]}
    state = {
        "participants": {"a": part("a", now), "b": part("b", now)},
        "heartbeats": {"a": now, "b": now},
        "prev_quorum": prev,
    }
    members, reason = C.quorum_compute(now, state, min_replicas=1, join_timeout_ms=60000)
    assert "Fast quorum found!" in reason
    assert [m["replica_id"] for m in members] == ["a", "b"]

    # a newcomer is admitted by the fast path without waiting
    state["participants"]["c"] = part("c", now)
    state["heartbeats"]["c"] = now
    members, reason = C.quorum_compute(now, state, min_replicas=1, join_timeout_ms=60000)
    assert "Fast quorum found!" in reason
    assert [m["replica_id"] for m in members] == ["a", "b", "c"]

    # a previous member is missing: no fast path, b still heartbeats without asking
    del state["participants"]["b"]
    members, reason = C.quorum_compute(now, state, min_replicas=1, join_timeout_ms=60000)
    assert members is None
    assert "waiting for 1 healthy but not participating stragglers" in reason


def test_shrink_only_keeps_previous_members():
    now = 7.0
    prev = {"quorum_id": 3, "participants": [member("a"), member("b")]}
    state = {
        "participants": {
            "a": part("a", now, shrink_only=True),
            "b": part("b", now),
            "c": part("c", now),
        },
        "heartbeats": {"a": now, "b": now, "c": now},
        "prev_quorum": prev,
    }
    members, reason = C.quorum_compute(now, state, min_replicas=1, join_timeout_ms=0)
    assert [m["replica_id"] for m in members] == ["a", "b"]
    assert "[shrink_only=true]" in reason


def test_split_brain_needs_majority_of_heartbeating():
    now = 9.0
    state = {
        "participants": {"a": part("a", now)},
        "heartbeats": {"a": now, "b": now, "c": now},
        "prev_quorum": None,
    }
    members, reason = C.quorum_compute(now, state, min_replicas=1, join_timeout_ms=0)
    assert members is None
    assert "New quorum not ready, only have 1 participants, need at least half of 3 healthy workers" in reason

    state["participants"]["b"] = part("b", now)
    members, reason = C.quorum_compute(now, state, min_replicas=1, join_timeout_ms=0)
    assert members is not None and len(members) == 2


def test_quorum_changed_only_looks_at_replica_ids():
    a = [member("a", step=1), member("b", step=1)]
    b = [member("a", step=5, addr="other"), member("b", step=7)]
    assert not C.quorum_changed(a, b)
    assert C.quorum_changed(a, [member("a"), member("c")])
    assert C.quorum_changed(a, [member("a")])


def test_results_first_step_everyone_heals_from_primary():
    members = [member("replica_0", step=0), member("replica_1", step=0)]
    r0 = C.compute_quorum_results("replica_0", 0, 1, members)
    assert not r0.heal
    assert r0.replica_rank == 0 and r0.replica_world_size == 2
    assert r0.recover_src_rank is None
    assert r0.recover_dst_ranks == [1]
    assert r0.max_step == 0 and r0.max_rank == 0 and r0.max_world_size == 2
    assert r0.store_address == "store_replica_0"

    r1 = C.compute_quorum_results("replica_1", 0, 1, members)
    assert r1.heal
    assert r1.recover_src_rank == 0
    assert r1.recover_src_manager_address == "addr_replica_0"
    assert r1.recover_dst_ranks == []
    assert r1.max_rank == 1

    # local rank 1 uses the second member as primary
    r = C.compute_quorum_results("replica_0", 1, 1, members)
    assert r.heal and r.recover_src_rank == 1 and r.store_address == "store_replica_1"
    r = C.compute_quorum_results("replica_1", 1, 1, members)
    assert not r.heal and r.recover_dst_ranks == [0]


def test_results_recovery_round_robin():
    steps = [0, 1, 0, 1, 0]
    members = [member(f"replica_{i}", step=s) for i, s in enumerate(steps)]
    r = C.compute_quorum_results("replica_0", 0, 1, members)
    assert r.heal and r.recover_src_rank == 1 and r.max_rank is None and r.max_world_size == 2
    assert r.max_step == 1 and r.replica_rank == 0 and r.replica_world_size == 5
    assert r.store_address == "store_replica_1"

    r = C.compute_quorum_results("replica_1", 0, 1, members)
    assert not r.heal and r.recover_dst_ranks == [0, 4] and r.max_rank == 0
    r = C.compute_quorum_results("replica_3", 0, 1, members)
    assert not r.heal and r.recover_dst_ranks == [2] and r.max_rank == 1

    # local rank 1 shifts the assignment and the primary store
    r = C.compute_quorum_results("replica_1", 1, 1, members)
    assert r.recover_dst_ranks == [2]
    assert r.store_address == "store_replica_3"
    r = C.compute_quorum_results("replica_3", 1, 1, members)
    assert r.recover_dst_ranks == [0, 4]


def test_results_unknown_replica():
    with pytest.raises(RuntimeError, match="not participating in returned quorum"):
        C.compute_quorum_results("nope", 0, 1, [member("a")])


def test_parse_grpc_timeout():
    assert C.parse_grpc_timeout("1H") == 3600.0
    assert C.parse_grpc_timeout("2M") == 120.0
    assert C.parse_grpc_timeout("3S") == 3.0
    assert C.parse_grpc_timeout("250m") == 0.25
    assert abs(C.parse_grpc_timeout("5u") - 5e-6) < 1e-12
    assert abs(C.parse_grpc_timeout("7n") - 7e-9) < 1e-15
    assert C.parse_grpc_timeout("") is None
    assert C.parse_grpc_timeout("12") is None
    assert C.parse_grpc_timeout("x5S") is None
    assert C.parse_grpc_timeout("123456789S") is None  # more than 8 digits


def test_retry_backoff():
    ok, attempts = C.retry_backoff_probe(fail_times=3, initial_ms=1)
    assert ok and attempts == 4
    ok, attempts = C.retry_backoff_probe(fail_times=100, initial_ms=1, max_retries=2)
    assert not ok and attempts == 3
    ok, attempts = C.retry_backoff_probe(fail_times=10**6, initial_ms=5, timeout_ms=50)
    assert not ok and attempts >= 2


# ------------------------------------------------------------------ property checks
def test_results_invariants_hold_for_random_quorums():
    """Whatever the steps of the members, the per-replica views of one quorum fit together:
    ranks are a permutation, recovery sources are up to date, and every replica that is behind is
    assigned to exactly one source."""
    from hypothesis import given, settings
    from hypothesis import strategies as st

    @settings(max_examples=200, deadline=None)
    @given(steps=st.lists(st.integers(min_value=0, max_value=3), min_size=1, max_size=9), local_rank=st.integers(0, 7))
    def check(steps, local_rank):
        members = [member(f"replica_{i:02d}", step=s) for i, s in enumerate(steps)]
        n = len(members)
        views = [C.compute_quorum_results(m["replica_id"], local_rank, 1, members) for m in members]
        max_step = max(steps)
        cohort = [i for i, s in enumerate(steps) if s == max_step]
        assert sorted(v.replica_rank for v in views) == list(range(n))
        primary = cohort[local_rank % len(cohort)]
        assigned = []
        for i, v in enumerate(views):
            assert v.replica_world_size == n and v.max_step == max_step and v.max_world_size == len(cohort)
            assert v.store_address == members[primary]["store_address"]
            in_cohort = i in cohort
            assert (v.max_rank is not None) == in_cohort
            if in_cohort:
                assert v.max_rank == cohort.index(i)
            # at step 0 everybody but the primary takes the primary's weights; later only the stragglers heal
            expect_heal = (i != primary) if max_step == 0 else not in_cohort
            assert v.heal == expect_heal, (steps, local_rank, i)
            if v.heal:
                assert v.recover_src_rank is not None and v.recover_src_rank in cohort
                assert v.recover_src_manager_address == members[v.recover_src_rank]["address"]
                assert v.recover_dst_ranks == []
            assigned.extend((dst, i) for dst in v.recover_dst_ranks)
        healing = sorted(i for i, v in enumerate(views) if v.heal)
        assert sorted(dst for dst, _ in assigned) == healing  # each exactly once
        for dst, src in assigned:
            assert views[dst].recover_src_rank == src

    check()


def test_quorum_compute_invariants_hold_for_random_states():
    """Safety properties of the lighthouse rule on random states: a quorum is sorted, made of healthy
    requesters only, at least ``min_replicas`` large, a strict majority of the heartbeating replicas,
    and never grows when a member of the previous quorum asked to shrink only."""
    from hypothesis import given, settings
    from hypothesis import strategies as st

    ids = [f"r{i}" for i in range(6)]
    replica = st.fixed_dictionaries({
        "asks": st.booleans(), "beats": st.booleans(), "beat_age": st.floats(0.0, 8.0), "joined_ago": st.floats(0.0, 3.0),
        "shrink_only": st.booleans(), "in_prev": st.booleans(),
    })

    @settings(max_examples=300, deadline=None)
    @given(spec=st.lists(replica, min_size=1, max_size=6), min_replicas=st.integers(1, 4), join_ms=st.sampled_from([0, 1000, 60000]))
    def check(spec, min_replicas, join_ms):
        now = 1000.0
        state = {"participants": {}, "heartbeats": {}, "prev_quorum": None}
        prev = []
        for rid, s in zip(ids, spec):
            if s["beats"]:
                state["heartbeats"][rid] = now - s["beat_age"]
            if s["asks"]:
                state["participants"][rid] = part(rid, now - s["joined_ago"], shrink_only=s["shrink_only"])
                state["heartbeats"].setdefault(rid, now)  # a request counts as a heartbeat
            if s["in_prev"]:
                prev.append(member(rid))
        if prev:
            state["prev_quorum"] = {"quorum_id": 1, "participants": prev}
        members, reason = C.quorum_compute(now, state, min_replicas=min_replicas, join_timeout_ms=join_ms, heartbeat_timeout_ms=5000)
        assert isinstance(reason, str) and reason
        if members is None:
            return
        got = [m["replica_id"] for m in members]
        healthy = {rid for rid, t in state["heartbeats"].items() if now - t < 5.0}
        assert got == sorted(got) and len(set(got)) == len(got)
        assert set(got) <= set(state["participants"]) & healthy
        if "Fast quorum" in reason:
            # every member of the previous quorum is back: accepted at once (with any newcomers), ahead of the
            # size rules, which that quorum satisfied when it formed
            assert {m["replica_id"] for m in prev} <= set(got)
        else:
            assert len(got) >= min_replicas
            assert len(got) > len(healthy) / 2  # split-brain guard: a strict majority of the heartbeating replicas
        shrink = any(state["participants"][rid]["member"]["shrink_only"] for rid in got)
        if shrink and prev:
            assert set(got) <= {m["replica_id"] for m in prev}

    check()
