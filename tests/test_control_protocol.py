"""Legacy control protocol (golden strings), registry, daemon core, token bucket."""
import math

import pytest


def test_parse_size_binary_suffixes(ctl):
    assert ctl.parse_size("64") == 64
    assert ctl.parse_size("128K") == 128 << 10
    assert ctl.parse_size("4M") == 4 << 20
    assert ctl.parse_size("2G") == 2 << 30
    assert ctl.parse_size("1GiB") == 1 << 30
    assert ctl.parse_size("x") is None and ctl.parse_size("") is None and ctl.parse_size("12Q") is None
    assert ctl.parse_size("99999999999999999999999") is None


def test_percentile_linear_interpolation(ctl):
    v = [10.0, 20.0, 30.0, 40.0]
    assert ctl.percentile(v, 0.5) == pytest.approx(25.0)
    assert ctl.percentile(v, 0.0) == 10.0 and ctl.percentile(v, 1.0) == 40.0
    assert ctl.percentile(v, 0.99) == pytest.approx(39.7)
    assert ctl.percentile([], 0.5) == 0.0


def test_legacy_replies_are_byte_exact(ctl):
    s = ctl.ControlState()
    s.configure(0, 100)
    s.enable()
    tail = "high_sleep_us=0 low1_sleep_us=100 low2_sleep_us=125 low3_sleep_us=150 low4_sleep_us=175"
    assert s.handle("STATUS\n") == f"OK mode=HIGH sleep_us=0 {tail} commands=0 stop=0\n"
    assert s.handle("LOW") == f"OK mode=LOW1 sleep_us=100 {tail} commands=1 stop=0\n"
    assert s.handle("  LOW3 \r\n") == f"OK mode=LOW3 sleep_us=150 {tail} commands=2 stop=0\n"
    assert s.handle("SLEEP 42") == f"OK mode=CUSTOM sleep_us=42 {tail} commands=3 stop=0\n"
    assert s.handle("STATUS") == f"OK mode=CUSTOM sleep_us=42 {tail} commands=3 stop=0\n"      # STATUS is not counted
    assert s.handle("bogus") == f"ERR unknown_cmd mode=CUSTOM sleep_us=42 {tail} commands=3 stop=0\n"
    assert s.handle("   ") == f"ERR empty mode=CUSTOM sleep_us=42 {tail} commands=3 stop=0\n"
    assert s.handle("STOP") == f"OK mode=CUSTOM sleep_us=42 {tail} commands=4 stop=1\n"
    assert s.handle("HIGH") == f"OK mode=HIGH sleep_us=0 {tail} commands=5 stop=1\n"
    assert s.stop_requested and s.mode == 1


def test_ladder_presets_can_be_overridden(ctl):
    s = ctl.ControlState()
    s.configure(5, 200, low2_us=300, low4_us=1000)
    s.enable()
    assert "low2_sleep_us=300 low3_sleep_us=300 low4_sleep_us=1000" in s.handle("STATUS")
    assert "sleep_us=5 " in s.handle("HIGH")


def test_ladder_fraction_follows_the_sleep_ladder(ctl):
    f1 = 0.5
    assert ctl.ladder_fraction(1, f1) == 1.0
    assert ctl.ladder_fraction(2, f1) == pytest.approx(0.5)
    assert ctl.ladder_fraction(3, f1) == pytest.approx(1 / 2.25)
    assert ctl.ladder_fraction(5, f1) == pytest.approx(1 / 2.75)
    assert [ctl.next_protect_mode(m) for m in (1, 2, 3, 4, 5, 0, 6)] == [2, 3, 4, 5, 5, 1, 1]


def _core(ctl, **kw):
    cfg = ctl.DaemonConfig()
    cfg.page_dir = ""            # pages on the heap: no files
    cfg.capacity_gbps = 64.0
    cfg.window_ns = 5_000_000
    for k, v in kw.items():
        setattr(cfg, k, v)
    return ctl.DaemonCore(cfg)


def test_register_budget_unregister(ctl):
    d = _core(ctl)
    r = d.handle_line("REGISTER kv_transfer high 40 kv_transfer", 0)
    assert r.startswith("OK flow_id=1 page=- lease_ms=5000 window_us=5000")
    assert d.handle_line("REGISTER kv_offload besteffort 0", 0).startswith("OK flow_id=2")
    assert d.handle_line("REGISTER x bad 1", 0) == "ERR bad_priority\n"
    assert d.handle_line("REGISTER x high nan", 0) == "ERR bad_target\n"
    assert d.handle_line("REGISTER x", 0).startswith("ERR usage")
    flows = d.handle_line("FLOWS", 0)
    assert flows.startswith("OK n=2 1:kv_transfer:100:40:kv_transfer:HIGH 2:kv_offload:0:0:kv_offload:HIGH")
    assert d.handle_line("BUDGET 2", 0).startswith("OK flow_id=2 mode=HIGH budget_gbps=-1")
    assert d.handle_line("BUDGET 9", 0) == "ERR unknown_flow\n"
    assert d.handle_line("UNREGISTER 2", 0) == "OK\n" and d.n_flows == 1
    assert d.handle_line("nonsense", 0) == "ERR unknown_cmd\n"
    assert d.handle_line("POLICY ladder", 0) == "OK policy=ladder\n" and d.policy_name == "ladder"
    assert d.handle_line("POLICY nope", 0) == "ERR unknown_policy\n"
    assert d.handle_line("WINDOW 1000", 0) == "OK window_us=1000\n"
    assert d.handle_line("WINDOW 5", 0) == "ERR bad_window\n"


def test_window_step_writes_grants_and_reserves_for_the_protected_flow(ctl):
    d = _core(ctl)
    d.handle_line("REGISTER kv_transfer high 40", 0)
    d.handle_line("REGISTER kv_offload besteffort 0", 0)
    win = 5_000_000
    # nothing to protect: both unlimited
    logs = d.step_window(win)
    assert [l.budget_bytes for l in logs] == [-1.0, -1.0]
    assert d.page_fields(2)["unlimited"] == 1 and d.page_fields(2)["epoch"] == 1
    # the protected flow has backlog, the best-effort flow is eating the link
    d.report_usage(1, 0, 0, 400_000_000)
    d.report_usage(2, 320_000_000, 320_000_000, 1 << 40)
    logs = d.step_window(2 * win)
    off = [l for l in logs if l.flow == "kv_offload"][0]
    assert off.decision in ("RESERVE", "DECREASE") and off.budget_bytes == pytest.approx((64 - 40) * 1e9 * 0.005, rel=0.6)
    f = d.page_fields(2)
    assert f["unlimited"] == 0 and f["granted_bytes"] > 320_000_000 and f["epoch"] == 2
    assert d.page_fields(1)["unlimited"] == 1
    # protected flow drains: release in one window
    d.report_usage(1, 400_000_000, 400_000_000, 0)
    logs = d.step_window(3 * win)
    assert d.page_fields(2)["unlimited"] == 1
    assert logs[1].csv().count(",") == ctl.DaemonCore.csv_header().count(",")


def test_manual_override_pins_a_flow_until_high(ctl):
    d = _core(ctl)
    d.handle_line("REGISTER kv_offload besteffort 0", 0)
    rep = d.handle_line("FLOW 1 LOW2", 0)
    assert rep.startswith("OK mode=LOW2 sleep_us=125")
    logs = d.step_window(5_000_000)
    assert logs[0].decision == "MANUAL" and logs[0].budget_bytes == pytest.approx(64e9 * 0.005 / 2.25, rel=1e-6)
    assert d.handle_line("FLOW 1 STOP", 0).endswith("stop=1\n") and d.page_fields(1)["stop"] == 1
    d.handle_line("FLOW 1 HIGH", 0)
    assert d.step_window(10_000_000)[0].decision != "MANUAL"
    assert d.handle_line("FLOW 7 HIGH", 0) == "ERR unknown_flow\n"


def test_leases_expire_and_renew(ctl):
    d = _core(ctl, lease_ns=1_000_000_000)
    d.handle_line("REGISTER a high 10", 0)
    d.handle_line("REGISTER b low 0", 0)
    assert d.handle_line("RENEW 1", 900_000_000) == "OK\n"
    d.step_window(1_100_000_000)            # b's lease (deadline 1.0 s) ran out, a's was renewed to 1.9 s
    assert d.n_flows == 1 and d.expired == 1
    assert d.handle_line("RENEW 2", 1_100_000_000) == "ERR unknown_flow\n"
    d.step_window(2_000_000_000)
    assert d.n_flows == 0 and d.expired == 2


def test_snapshot_restore_round_trip(ctl, tmp_path):
    d = _core(ctl, page_dir=str(tmp_path), tag="t")
    d.keep_pages_on_exit(True)
    d.handle_line("REGISTER kv_transfer high 40", 0)
    d.handle_line("REGISTER kv_offload besteffort 0", 0)
    d.handle_line("POLICY ladder", 0)
    d.report_usage(1, 0, 0, 1 << 30)
    d.report_usage(2, 10, 10, 1 << 40)
    d.step_window(5_000_000)
    snap = d.snapshot_json()
    assert '"policy":"ladder"' in snap and '"name":"kv_offload"' in snap
    granted = d.page_fields(2)["granted_bytes"]
    del d
    d2 = _core(ctl, page_dir=str(tmp_path), tag="t")
    assert d2.restore_json(snap, 0) and d2.n_flows == 2 and d2.policy_name == "ladder"
    assert d2.page_fields(2)["granted_bytes"] == granted       # the page survived the daemon
    assert d2.handle_line("REGISTER c low 0", 0).startswith("OK flow_id=3")
    assert not d2.restore_json("{}", 0)


def test_token_bucket(ctl):
    b = ctl.TokenBucket()
    b.burst_windows = 2.0
    w = 5_000_000
    assert b.refill(10.0, w, 0) == 50_000_000
    assert b.refill(10.0, w, 0) == 100_000_000           # one window of unused credit may be carried
    assert b.refill(10.0, w, 0) == 100_000_000           # ... but not more than burst_windows
    assert b.refill(10.0, w, 100_000_000) == 150_000_000  # all spent: one more window
    assert b.refill(10.0, w, 170_000_000) == 200_000_000  # tickets beyond the grant are waiting, not spent
    assert b.refill(-1.0, w, 0) == 200_000_000            # unlimited leaves the counter alone
    g = b.refill(1.0, w, 200_000_000)
    assert g == 205_000_000 and b.refill(0.0, w, 205_000_000) == 205_000_000


def test_heartbeat_rule_of_host_data_paths(ctl):
    """A page carries the daemon's heartbeat contract; a host data path that sees the epoch stand still for
    dead_after_windows windows follows dead_policy: stall on the last grant, run unpaced, or grant itself a static rate."""
    win = 1_000_000
    for policy, name in ((0, "stall"), (1, "unpaced"), (2, "static")):
        d = _core(ctl, window_ns=win, dead_after_windows=4, dead_policy=policy, dead_fallback_gbps=2.0, policy="static")
        d.handle_line("REGISTER kv_offload besteffort 0 kv_offload", 0)
        d.handle_line("FLOW 1 LOW1", 0)
        d.report_usage(1, 0, 0, 1 << 30)
        d.step_window(win)
        d.step_window(2 * win)
        f = d.page_fields(1)
        assert f["dead_after_windows"] == 4 and f["dead_policy"] == policy and f["fallback_per_window"] == 2_000_000
        granted = f["granted_bytes"]
        assert f["unlimited"] == 0 and granted > 0
        w = ctl.HeartbeatWatch()
        assert w.allowance(d, 1, 10 * win) == granted                     # first look starts the watch
        d.step_window(11 * win)
        g2 = d.page_fields(1)["granted_bytes"]
        assert w.allowance(d, 1, 12 * win) == g2 and w.t_dead_ns == 0     # the epoch moved: alive
        assert w.allowance(d, 1, 16 * win) == g2                          # 4 windows of silence: not yet over the line
        got = w.allowance(d, 1, 17 * win)                                 # now it is
        assert w.t_dead_ns == 17 * win and d.page_fields(1)["heartbeat_lost"] == d.page_fields(1)["epoch"] + 1, name
        if name == "stall":
            assert got == g2 and w.allowance(d, 1, 100 * win) == g2
        elif name == "unpaced":
            assert got == 2**64 - 1
        else:
            assert got == g2 and w.allowance(d, 1, 27 * win) == g2 + 10 * 2_000_000
        d.step_window(30 * win)                                           # the daemon is back: grants rule again
        assert w.allowance(d, 1, 31 * win) == d.page_fields(1)["granted_bytes"] and w.t_dead_ns == 0


def test_protocol_survives_arbitrary_lines(ctl):
    """Property test: whatever line arrives (control characters, huge numbers, half commands, many tokens), the daemon core
    answers with exactly one line that starts with OK or ERR, stays consistent (flow count bounded by the registrations it
    accepted, grants never decrease) and keeps answering afterwards. The reference's end point gets its robustness from reading
    at most 255 bytes and knowing eight words (src/cpu_client.cc:176-236,299-300); this one has a grammar, so it is fuzzed."""
    from hypothesis import given, settings
    from hypothesis import strategies as st

    words = st.sampled_from(["REGISTER", "RENEW", "UNREGISTER", "BUDGET", "FLOWS", "FLOW", "POLICY", "WINDOW", "CAPACITY", "PING", "STATUS", "HIGH",
                             "LOW", "LOW1", "LOW2", "LOW3", "LOW4", "SLEEP", "STOP", "kv_transfer", "kv_offload", "high", "low", "besteffort",
                             "nan", "inf", "-1", "0", "1", "2", "40", "1e308", "99999999999999999999", "target_track", "weighted_track", "ladder", "static", "none", "x",
                             "LINK", "LINKS", "STATS", "link=default", "link=nv", "link=", "nv", "default", "700"])
    junk = st.text(alphabet=st.characters(blacklist_categories=("Cs",), blacklist_characters="\n"), max_size=40)
    line = st.one_of(st.lists(st.one_of(words, junk), max_size=8).map(" ".join), junk)

    d = _core(ctl, window_ns=1_000_000)
    state = {"now": 0, "granted": {}}

    @settings(max_examples=400, deadline=None)
    @given(line)
    def check(text):
        state["now"] += 1_000_000
        reply = d.handle_line(text, state["now"])
        assert reply.endswith("\n") and reply.count("\n") == 1 and (reply.startswith("OK") or reply.startswith("ERR")), (text, reply)
        d.step_window(state["now"])
        assert 0 <= d.n_flows <= 4096
        flows = d.handle_line("FLOWS", state["now"])
        assert flows.startswith("OK n=")
        for tok in flows.split()[2:]:
            fid = int(tok.split(":")[0])
            g = d.page_fields(fid)["granted_bytes"]
            assert g >= state["granted"].get(fid, 0), (text, fid)
            state["granted"][fid] = g
        assert d.handle_line("PING", state["now"]).startswith("OK")
        links = d.handle_line("LINKS", state["now"])
        assert links.startswith("OK n=") and " default:" in links and d.link_count <= 64

    check()


def test_window_step_cost_leaves_room_in_a_one_millisecond_window(ctl):
    """256 registered flows, all with traffic: one policy + grant pass must take a small part of the shortest window (1 ms).
    The reference's loop polls every 100 ms from Python (src/tools/pcie_case_study_controller.py:148)."""
    import time

    d = _core(ctl, window_ns=1_000_000, policy="target_track")
    for i in range(256):
        prio, target = ("high", 1.0) if i % 8 == 0 else ("besteffort", 0.0)
        assert d.handle_line(f"REGISTER f{i} {prio} {target} kind{i % 4}", 0).startswith("OK")
    now = 0
    for w in range(50):                                              # settle
        now += 1_000_000
        for i in range(1, 257):
            d.report_usage(i, w * 100_000, w * 100_000, 1 << 20)
        d.step_window(now)
    best = float("inf")
    for _ in range(5):                                               # best of five batches: a busy host only ever adds time
        t0 = time.perf_counter()
        n = 100
        for w in range(n):
            now += 1_000_000
            d.step_window(now)
        best = min(best, (time.perf_counter() - t0) / n * 1e6)
    assert best < 250.0, best                                        # a quarter of the shortest window, with 256 flows


def test_native_page_pacer_grants_at_its_rate_and_lets_a_flow_catch_up(ctl):
    """The in-process pacer is a native thread on a page given by address: it grants rate x time while the flow keeps up, holds
    the grant a couple of windows ahead of a flow that does not, and bumps the epoch every window (the heartbeat)."""
    import ctypes
    import time

    page = (ctypes.c_uint64 * 32)()                  # 256 bytes; [1] granted, [2] epoch, [16] consumed
    pacer = ctl.PagePacer(ctypes.addressof(page), 1.0, 1_000_000, 2.0)        # 1 GB/s, 1 ms windows
    pacer.start(0)
    time.sleep(0.05)
    idle = page[1]
    assert 0 < idle < 6_000_000                      # nothing consumed: the grant stays about two windows ahead
    t0 = time.perf_counter()
    g0 = page[1]
    for _ in range(60):                              # a flow that uses every byte it is given
        page[16] = page[1]
        time.sleep(0.001)
    dt = time.perf_counter() - t0
    pacer.stop()
    rate = (page[1] - g0) / dt / 1e9
    assert 0.7 < rate < 1.3, rate
    assert page[2] >= pacer.windows > 50 and page[5] & 0xffffffff00000000 == 0      # epoch per window; `unlimited` (high half of word 5) off


def test_flows_on_different_links_do_not_take_bandwidth_from_one_another(ctl):
    """Links: each is one shared capacity with its own policy pass. A protected NVLink flow must throttle the best-effort
    flow that shares its link and leave alone the one on the PCIe link, whatever that one is doing."""
    d = _core(ctl, capacity_gbps=64.0)
    assert d.handle_line("LINKS", 0) == "OK n=1 default:64\n"
    assert d.handle_line("LINK nvlink:gpu0 700", 0) == "OK link=nvlink:gpu0 capacity_gbps=700.000 flows=0\n"
    assert d.handle_line("LINK bad/name 10", 0) == "ERR bad_link_name\n"
    assert d.handle_line("LINK nvlink:gpu0 -5", 0) == "ERR bad_capacity\n"
    assert d.handle_line("LINK nope", 0) == "ERR unknown_link\n"
    assert d.handle_line("REGISTER x high 1 link=nope", 0) == "ERR unknown_link\n" and d.n_flows == 0
    assert d.handle_line("REGISTER kv_transfer high 600 link=nvlink:gpu0", 0).rstrip().endswith("link=nvlink:gpu0")
    assert d.handle_line("REGISTER kv_bursts besteffort 0 kv_transfer link=nvlink:gpu0", 0).startswith("OK flow_id=2")
    assert d.handle_line("REGISTER kv_offload besteffort 0", 0).rstrip().endswith("link=default")       # PCIe: the default link
    assert d.handle_line("LINK nvlink:gpu0", 0) == "OK link=nvlink:gpu0 capacity_gbps=700.000 flows=2\n"
    assert d.handle_line("FLOWS", 0).split()[2:] == ["1:kv_transfer:100:600:kv_transfer:HIGH:nvlink:gpu0",
                                                     "2:kv_bursts:0:0:kv_transfer:HIGH:nvlink:gpu0", "3:kv_offload:0:0:kv_offload:HIGH"]
    win = 5_000_000
    d.step_window(win)
    # the protected flow has backlog; both best-effort flows run flat out on their own links
    d.report_usage(1, 0, 0, 4_000_000_000)
    d.report_usage(2, 3_400_000_000, 3_400_000_000, 1 << 40)          # 680 GB/s on the NVLink link
    d.report_usage(3, 300_000_000, 300_000_000, 1 << 40)              # 60 GB/s on the 64 GB/s default link
    logs = {l.flow: l for l in d.step_window(2 * win)}
    assert logs["kv_bursts"].decision in ("RESERVE", "DECREASE")
    assert logs["kv_bursts"].budget_bytes == pytest.approx((700 - 600) * 1e9 * 0.005, rel=0.6)           # what the link has left
    assert logs["kv_offload"].budget_bytes == -1.0 and d.page_fields(3)["unlimited"] == 1               # other link: untouched
    assert logs["kv_bursts"].link_util_pct == pytest.approx(100 * 680 / 700, rel=0.02)
    assert logs["kv_offload"].link_util_pct == pytest.approx(100 * 60 / 64, rel=0.02)
    stats = dict(kv.split("=", 1) for kv in d.handle_line("STATS", 0).split()[1:])
    assert stats["windows"] == "2" and stats["flows"] == "3" and stats["links"] == "2" and stats["policy"] == "target_track"
    assert float(stats["util_pct:nvlink:gpu0"]) == pytest.approx(100 * 680 / 700, rel=0.02) and float(stats["util_pct:default"]) > 90
    assert 0 < float(stats["step_us_last"]) <= float(stats["step_us_max"]) < 5000
    # capacity of a link can be changed while flows run; the default link follows CAPACITY as before
    assert d.handle_line("LINK nvlink:gpu0 900", 0).startswith("OK link=nvlink:gpu0 capacity_gbps=900.000 flows=2")
    assert d.handle_line("CAPACITY 32", 0) == "OK capacity_gbps=32.000\n" and d.handle_line("LINKS", 0) == "OK n=2 default:32 nvlink:gpu0:900\n"
    # snapshot and restore keep links and membership
    d2 = _core(ctl)
    assert d2.restore_json(d.snapshot_json(), 0)
    assert d2.handle_line("LINKS", 0) == "OK n=2 default:32 nvlink:gpu0:900\n"
    assert d2.handle_line("LINK nvlink:gpu0", 0).endswith("flows=2\n")
    assert "3:kv_offload:0:0:kv_offload:HIGH" in d2.handle_line("FLOWS", 0) and "2:kv_bursts:0:0:kv_transfer:CUSTOM:nvlink:gpu0" in d2.handle_line("FLOWS", 0)   # throttled when the snapshot was taken


def test_measured_link_traffic_replaces_the_sum_over_registered_flows(ctl):
    """Traffic that never registered (another job's copies on the same PCIe link) is invisible in the flows' counters; with a
    measured figure for the link, the ladder policy sees the link as busy and protects the restore flow."""
    d = _core(ctl, policy="ladder")
    d.handle_line("LINK pcie:gpu0 55", 0)
    d.handle_line("REGISTER restore high 30 link=pcie:gpu0", 0)
    d.handle_line("REGISTER offload besteffort 0 link=pcie:gpu0", 0)
    win = 5_000_000
    d.step_window(win)
    for k in range(2, 6):                                              # the restore gets 10 GB/s of its 30, the offload 5
        d.report_usage(1, k * 50_000_000, k * 50_000_000, 1 << 30)
        d.report_usage(2, k * 25_000_000, k * 25_000_000, 1 << 40)
        logs = d.step_window(k * win)                                   # by the flows' counters the link is a quarter busy
    assert all(l.link_util_pct < 40 for l in logs) and [l.decision for l in logs if l.flow == "offload"] == ["HOLD"]
    for k in range(6, 10):
        d.report_usage(1, k * 50_000_000, k * 50_000_000, 1 << 30)
        d.report_usage(2, k * 25_000_000, k * 25_000_000, 1 << 40)
        logs = d.step_window(k * win, 0.0, {"pcie:gpu0": 52.0})         # NVML says 52 of 55 GB/s are in use
    off = [l for l in logs if l.flow == "offload"][0]
    assert off.link_util_pct == pytest.approx(100 * 52 / 55) and off.mode != 1                 # escalated out of HIGH
    assert d.step_window(10 * win, 0.0, {"other": 1.0})[0].link_util_pct < 40                  # names that match no link are ignored
