"""Policies as state machines, the fabric simulator, the config-1 experiment, workload generators."""
import math

import pytest


def _sig(ctl, id, prio, target, inst, smooth, backlog):
    s = ctl.FlowSignal()
    s.id, s.priority, s.target_gbps, s.inst_gbps, s.smooth_gbps, s.backlog_bytes = id, prio, target, inst, smooth, backlog
    s.active = backlog > 0 or inst > 0
    return s


def _link(ctl, util, cap=64.0):
    l = ctl.LinkSignal()
    l.capacity_gbps, l.util_pct = cap, util
    return l


def test_ladder_policy_trace(ctl):
    """HIGH -> LOW1 -> ... -> LOW4, never back while the protected flow is unfinished, HIGH when it is done."""
    cfg = ctl.PolicyConfig()
    p = ctl.make_policy("ladder", cfg)
    kv = lambda smooth, backlog: _sig(ctl, 1, 100, 40.0, smooth, smooth, backlog)
    off = _sig(ctl, 2, 0, 0.0, 30.0, 30.0, 1 << 40)
    seq = []
    for smooth, util, backlog in [(20, 99, 1), (20, 99, 1), (35, 99, 1), (20, 50, 1), (20, 99, 1), (20, 99, 1), (20, 99, 1),
                                  (39, 99, 1), (0, 10, 0), (0, 10, 0)]:
        d = p.step([kv(smooth, backlog), off], _link(ctl, util))
        seq.append((ctl.mode_name(d[1].mode), d[1].decision))
    assert seq == [("LOW1", "SWITCH_LOW1"), ("LOW2", "ESCALATE_LOW2"), ("LOW2", "HOLD"),      # 35 >= 0.65*40: not bad
                   ("LOW2", "HOLD"),                                                           # link not busy
                   ("LOW3", "ESCALATE_LOW3"), ("LOW4", "ESCALATE_LOW4"), ("LOW4", "HOLD"),     # top of the ladder
                   ("LOW4", "HOLD"),                                                           # healthy, but never de-escalates
                   ("HIGH", "RESTORE_DONE_HIGH"), ("HIGH", "HOLD")]
    d = p.step([kv(20, 1), off], _link(ctl, 99))
    assert d[0].budget_gbps == -1.0 and d[1].budget_gbps == pytest.approx(64 * 0.5)


def test_ladder_enter_windows_and_nan_signals(ctl):
    cfg = ctl.PolicyConfig()
    cfg.enter_windows = 3
    p = ctl.make_policy("ladder", cfg)
    kv = _sig(ctl, 1, 100, 40.0, 10, 10, 1)
    off = _sig(ctl, 2, 0, 0.0, 30.0, 30.0, 1)
    modes = [p.step([kv, off], _link(ctl, 99))[1].mode for _ in range(4)]
    assert modes == [1, 1, 2, 2]
    bad = _sig(ctl, 1, 100, 40.0, float("nan"), float("nan"), 1)
    p2 = ctl.make_policy("ladder", ctl.PolicyConfig())
    assert p2.step([bad, off], _link(ctl, 99))[1].mode == 1          # a missing signal never escalates
    assert p2.step([kv, off], _link(ctl, float("nan")))[1].mode == 1


def test_target_track_reserves_decreases_and_recovers(ctl):
    cfg = ctl.PolicyConfig()
    p = ctl.make_policy("target_track", cfg)
    off = _sig(ctl, 2, 0, 0.0, 30.0, 30.0, 1 << 40)
    idle = _sig(ctl, 1, 100, 40.0, 0, 0, 0)
    assert p.step([idle, off], _link(ctl, 50))[1].budget_gbps == -1.0
    busy = _sig(ctl, 1, 100, 40.0, 20, 20, 1 << 30)
    d = p.step([busy, off], _link(ctl, 99))                  # bad: below 0.65*40 with a busy link
    assert d[1].decision == "DECREASE" and d[1].budget_gbps == pytest.approx(24 * 0.5)
    d = p.step([busy, off], _link(ctl, 99))
    assert d[1].budget_gbps == pytest.approx(24 * 0.25)
    ok = _sig(ctl, 1, 100, 40.0, 39, 39, 1 << 30)             # above exit_ratio: healthy
    p.step([ok, off], _link(ctl, 99))
    d = p.step([ok, off], _link(ctl, 99))                     # exit_windows = 2 -> additive increase
    assert d[1].decision == "INCREASE" and d[1].budget_gbps == pytest.approx(24 * 0.30)
    d = p.step([idle, off], _link(ctl, 30))
    assert d[1].decision == "RELEASE" and d[1].budget_gbps == -1.0
    floor = ctl.make_policy("target_track", cfg)
    for _ in range(20):
        d = floor.step([busy, off], _link(ctl, 99))
    assert d[1].budget_gbps == pytest.approx(64 * cfg.min_be_fraction)   # never starved entirely


def test_none_and_static_policies(ctl):
    kv = _sig(ctl, 1, 100, 40.0, 20, 20, 1)
    off = _sig(ctl, 2, 0, 0.0, 30.0, 30.0, 1)
    assert [d.budget_gbps for d in ctl.make_policy("none").step([kv, off], _link(ctl, 99))] == [-1.0, -1.0]
    d = ctl.make_policy("static").step([kv, off], _link(ctl, 0))
    assert d[0].budget_gbps == -1.0 and d[1].mode == 2 and d[1].budget_gbps == pytest.approx(32.0)
    assert ctl.make_policy("always_high").name == "none"


def test_maxmin_fair(ctl):
    assert ctl.maxmin_fair([10, 10], 10) == pytest.approx([5, 5])
    assert ctl.maxmin_fair([2, 10, 10], 12) == pytest.approx([2, 5, 5])
    assert ctl.maxmin_fair([1, 1], 10) == pytest.approx([1, 1])
    assert ctl.maxmin_fair([0, 7], 5) == pytest.approx([0, 5])
    assert sum(ctl.maxmin_fair([3, 9, 27, 81], 50)) == pytest.approx(50)


def test_simulator_conserves_bytes_and_respects_capacity(ctl):
    from skygdr_b200.control.config1 import Config1, run_arm

    cfg = Config1(duration_s=2.0)
    for arm in ("always_high", "target_track", "ladder_100ms"):
        res = run_arm(cfg, arm)
        done = [r for r in res.requests if r.flow_id == 1 and r.finish_ms >= 0]
        assert len(done) == len([r for r in res.requests if r.flow_id == 1])          # every request finished
        assert sum(r.bytes for r in done) == pytest.approx(res.bytes_moved[0], rel=1e-6)
        assert res.bytes_moved[0] == pytest.approx(res.bytes_offered[0], rel=1e-6)
        assert res.link_bytes == pytest.approx(sum(res.bytes_moved), rel=1e-9)
        for r in res.rows:
            assert r.link_util_pct <= 100.0 + 1e-6
        assert all(r.finish_ms >= r.arrival_ms and r.start_ms >= r.arrival_ms - 1e-9 for r in done)
        assert res.windows >= 400 and len(res.rows) == 2 * res.windows


def test_config1_scheduling_beats_no_scheduling(ctl):
    from skygdr_b200.control.config1 import Config1, controller_csv, run_arm, run_config1

    out = run_config1(Config1())
    hi, tt, lo = out["always_high"], out["target_track"], out["always_low"]
    assert 150 <= hi["requests"] <= 250 and hi["unfinished"] == 0 and hi["windows"] >= 2000
    # the reference reports a 19.4-34.4 % flow-time reduction for its scheduled system (README.md:74)
    assert tt["flow_time_p50_ms"] < 0.85 * hi["flow_time_p50_ms"]
    assert tt["flow_time_p99_ms"] < 0.85 * hi["flow_time_p99_ms"]
    assert tt["offload_goodput_gbps"] > 0.9 * hi["offload_goodput_gbps"]         # ... without starving the offload
    assert lo["offload_goodput_gbps"] < 0.6 * hi["offload_goodput_gbps"]         # the static arm pays all the time
    assert out["ladder"]["flow_time_p50_ms"] <= out["ladder_100ms"]["flow_time_p50_ms"] + 1e-9
    csv = controller_csv(run_arm(Config1(duration_s=0.5), "target_track"))
    head = csv.splitlines()[0].split(",")
    assert head[:6] == ["t_ms", "window_id", "flow", "mode", "decision", "budget_bytes"]
    assert any(",RESERVE," in line or ",DECREASE," in line for line in csv.splitlines())


def test_simulation_is_deterministic(ctl):
    from skygdr_b200.control.config1 import Config1, run_arm, summarise

    a = summarise(Config1(duration_s=1.0), run_arm(Config1(duration_s=1.0), "target_track"))
    b = summarise(Config1(duration_s=1.0), run_arm(Config1(duration_s=1.0), "target_track"))
    assert a == b
    c = summarise(Config1(duration_s=1.0, seed=1), run_arm(Config1(duration_s=1.0, seed=1), "target_track"))
    assert c != a


def test_trace_sampler_matches_the_published_quantiles(ctl):
    for name, (p50, p90, p99, cap) in {"input": (63917, 114888, 166322, 200000), "cached": (60928, 112512, 162048, 200000),
                                       "computed": (758, 8736, 53323, 70000)}.items():
        xs = sorted(ctl.sample_trace_tokens(name, 1, 200000))
        q = lambda f: xs[int(f * (len(xs) - 1))]
        assert q(0.5) == pytest.approx(p50, rel=0.03) and q(0.9) == pytest.approx(p90, rel=0.03)
        assert q(0.99) == pytest.approx(p99, rel=0.05)
        assert xs[0] >= p50 // 8 and xs[-1] <= cap
    assert ctl.sample_trace_tokens("computed", 7, 50) == ctl.sample_trace_tokens("computed", 7, 50)
    assert ctl.sample_trace_tokens("computed", 7, 50) != ctl.sample_trace_tokens("computed", 8, 50)
    assert max(ctl.sample_trace_tokens("input", 1, 5000, 100000)) <= 166322      # the cap never drops below p99
    with pytest.raises(ValueError):
        ctl.sample_trace_tokens("nope", 1, 1)


def test_kv_bytes_and_poisson(ctl):
    assert ctl.kv_bytes_for_tokens(1, 36, 8, 128, 2) == 147456                 # Qwen3-8B: 144 KiB per token
    assert ctl.kv_bytes_for_tokens(1, 80, 8, 128, 2) == 327680
    assert ctl.kv_bytes_for_tokens(3, 1, 1, 5, 2) == 256                       # rounded up to 256 B
    arr = ctl.poisson_uniform(0, 20.0, 10.0, 50e6, 500e6)
    assert 150 <= len(arr) <= 250 and all(50e6 <= b <= 500e6 for _, b in arr)
    ts = [t for t, _ in arr]
    assert ts == sorted(ts) and ts[-1] < 10.0
    assert arr == ctl.poisson_uniform(0, 20.0, 10.0, 50e6, 500e6)
    rng = ctl.Rng(3)
    vals = [rng.lognormal(8192, 0.8, 1024, 32768) for _ in range(20000)]
    assert min(vals) >= 1024 and max(vals) <= 32768
    assert sorted(vals)[10000] == pytest.approx(8192, rel=0.05)


def test_contended_efficiency_costs_goodput_only_in_company(ctl):
    """A flow with contended_efficiency 0.9 (the reference's HBM-bound decoder next to an inbound copy) delivers 90 % of its
    link share while another flow is moving bytes and all of it when alone; the link time is spent either way."""
    def run(flows):
        cfg = ctl.SimConfig()
        cfg.capacity_gbps, cfg.duration_s, cfg.drain_s, cfg.policy = 64.0, 1.0, 0.0, "none"
        specs = []
        for name, eff in flows:
            s = ctl.SimFlowSpec()
            s.name, s.backlogged, s.contended_efficiency = name, True, eff
            specs.append(s)
        return ctl.run_simulation(cfg, specs)

    both = run([("copy", 1.0), ("decode", 0.9)])
    assert both.bytes_moved[0] == pytest.approx(32e9, rel=0.01) and both.bytes_moved[1] == pytest.approx(0.9 * 32e9, rel=0.01)
    assert both.link_bytes == pytest.approx(64e9, rel=0.01)                       # the link was busy all the time
    alone = run([("decode", 0.9)])
    assert alone.bytes_moved[0] == pytest.approx(64e9, rel=0.01)


def test_simulated_links_are_independent(ctl):
    """Two links in one simulation: the protected NVLink-like flow is shielded from the best-effort flow on its own link,
    and the best-effort flow on the other link keeps that link's full rate the whole time."""
    cfg = ctl.SimConfig()
    cfg.capacity_gbps, cfg.more_links_gbps, cfg.duration_s, cfg.drain_s, cfg.policy = 64.0, [700.0], 2.0, 1.0, "target_track"
    prot, be_same, be_other = ctl.SimFlowSpec(), ctl.SimFlowSpec(), ctl.SimFlowSpec()
    prot.name, prot.priority, prot.target_gbps, prot.link = "kv_transfer", 100, 600.0, 1
    prot.set_arrivals([(0.05 * k, 20_000_000_000) for k in range(1, 30)])      # 20 GB every 50 ms: 400 GB/s offered
    be_same.name, be_same.backlogged, be_same.link = "kv_bursts", True, 1
    be_other.name, be_other.backlogged, be_other.link = "kv_offload", True, 0
    res = ctl.run_simulation(cfg, [prot, be_same, be_other])
    assert res.bytes_moved[2] == pytest.approx(64e9 * 2.0, rel=0.01)          # the PCIe-like link never noticed
    ft = sorted(res.flow_times_ms(1))
    assert len(ft) == 29 and ft[len(ft) // 2] < 45.0                          # 20 GB at >= 600 GB/s is 33 ms; fair sharing would give 57 ms
    rows_same = [r for r in res.rows if r.flow == "kv_bursts"]
    assert any(r.budget_bytes >= 0 for r in rows_same)                        # it was throttled at times ...
    assert all(r.budget_bytes < 0 for r in res.rows if r.flow == "kv_offload")   # ... and the other link's flow never
    assert max(r.link_util_pct for r in res.rows if r.flow == "kv_offload") <= 100.0 + 1e-6
    # unscheduled, the same workload shares the fast link half and half while a request is in flight
    cfg.policy = "none"
    res0 = ctl.run_simulation(cfg, [prot, be_same, be_other])
    ft0 = sorted(res0.flow_times_ms(1))
    assert ft0[len(ft0) // 2] > ft[len(ft) // 2] * 1.2


def test_weighted_track_splits_the_unprotected_share_by_priority(ctl):
    """Two best-effort flows with priorities 10 and 0 next to a protected flow: while the protected flow is served they share
    what is left 11 : 1 (target_track gives them halves); alone on the link, priorities do not matter."""
    def run(policy):
        cfg = ctl.SimConfig()
        cfg.capacity_gbps, cfg.duration_s, cfg.drain_s, cfg.policy = 64.0, 2.0, 0.5, policy
        prot, a, b = ctl.SimFlowSpec(), ctl.SimFlowSpec(), ctl.SimFlowSpec()
        prot.name, prot.priority, prot.target_gbps, prot.backlogged = "kv_transfer", 100, 40.0, True     # always being served
        a.name, a.priority, a.backlogged = "offload_important", 10, True
        b.name, b.priority, b.backlogged = "offload_background", 0, True
        return ctl.run_simulation(cfg, [prot, a, b])

    w = run("weighted_track")
    assert w.bytes_moved[0] == pytest.approx(40e9 * 2.0, rel=0.1)                   # the protected flow gets its goal
    assert w.bytes_moved[1] / w.bytes_moved[2] == pytest.approx(11.0, rel=0.15)
    assert sum(w.bytes_moved) == pytest.approx(64e9 * 2.0, rel=0.05)                # nothing is wasted
    t = run("target_track")
    assert t.bytes_moved[1] / t.bytes_moved[2] == pytest.approx(1.0, rel=0.1)


def test_a_python_callable_can_be_the_simulator_policy(ctl):
    """A rule written in Python, tried against the simulator: hold the best-effort flow to a fixed 10 GB/s while the protected
    flow has backlog. It must behave like the equivalent built-in reservation and see sensible signals every window."""
    seen = {"windows": 0, "max_util": 0.0}

    def rule(flows, link):
        seen["windows"] += 1
        seen["max_util"] = max(seen["max_util"], link.util_pct)
        busy = any(f.target_gbps > 0 and f.backlog_bytes > 0 for f in flows)
        return [-1.0 if f.target_gbps > 0 else (10.0 if busy else -1.0) for f in flows]

    cfg = ctl.SimConfig()
    cfg.capacity_gbps, cfg.duration_s, cfg.drain_s = 64.0, 2.0, 1.0
    prot, be = ctl.SimFlowSpec(), ctl.SimFlowSpec()
    prot.name, prot.priority, prot.target_gbps = "kv_transfer", 100, 40.0
    prot.set_arrivals([(0.1 * k, 1_000_000_000) for k in range(1, 18)])          # 1 GB every 100 ms
    be.name, be.backlogged = "kv_offload", True
    res = ctl.run_simulation(cfg, [prot, be], policy=rule)
    assert seen["windows"] == res.windows and 99.0 < seen["max_util"] <= 100.0 + 1e-6
    ft = sorted(res.flow_times_ms(1))
    assert len(ft) == 17 and ft[len(ft) // 2] == pytest.approx(1e9 / 54e9 * 1e3, rel=0.25)    # 54 of 64 GB/s while it is in flight
    rows = [r for r in res.rows if r.flow == "kv_offload"]
    assert {r.decision for r in rows} == {"HOLD", "CALLBACK"} and any(r.budget_bytes == pytest.approx(10e9 * 0.005) for r in rows)
    none = ctl.run_simulation(cfg, [prot, be])                                   # by name, as before
    assert none.windows == res.windows
    with pytest.raises(Exception):
        ctl.run_simulation(cfg, [prot, be], policy=lambda flows, link: "not a list")
