"""The daemon under AddressSanitizer+UBSan and under ThreadSanitizer: concurrent clients, window timer, lease expiry,
shutdown. Any report makes the sanitizer exit non-zero or print to stderr."""
import os
import signal
import socket
import subprocess
import threading
import time

import pytest

from skygdr_b200 import build
from skygdr_b200.control import FabricClient, wait_for_control


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


@pytest.mark.parametrize("kind", ["address", "thread"])
def test_daemon_session_is_clean_under_sanitizer(kind, tmp_path):
    exe = build.build_sanitized(kind)
    port = _free_port()
    env = dict(os.environ, ASAN_OPTIONS="detect_leaks=1:abort_on_error=0", TSAN_OPTIONS="halt_on_error=0")
    p = subprocess.Popen([str(exe), "--port", str(port), "--window_us", "1000", "--lease_ms", "300", "--page_dir", str(tmp_path),
                          "--log", str(tmp_path / "w.csv"), "--link", "nvlink=700", "--unix", str(tmp_path / "d.sock"),
                          "--snapshot", str(tmp_path / "snap.json")], stderr=subprocess.PIPE, text=True, env=env)
    try:
        wait_for_control("127.0.0.1", port, 15.0, command="PING")

        def client(i):
            # half of the clients come over the Unix socket, a third of the flows live on the second link
            with (FabricClient(unix=str(tmp_path / "d.sock")) if i % 2 else FabricClient(port=port)) as c:
                f = c.register(f"flow{i}", "high" if i % 2 else "besteffort", 10.0 * (i % 2), link="nvlink" if i % 3 == 0 else None)
                for k in range(20):
                    f.report(k * 1_000_000, k * 1_000_000, 5_000_000 if i % 2 else 1 << 40)
                    c.renew(f)
                    c.budget(f)
                    c.request("STATS")
                    if k == 10 and i == 0:
                        c.link("late_link", 55.0)      # a link appears while windows are running
                    time.sleep(0.005)
                if i % 3:
                    c.unregister(f)            # the others are left to expire

        threads = [threading.Thread(target=client, args=(i,)) for i in range(6)]
        for t in threads:
            t.start()
        for t in threads:
            t.join()
        time.sleep(0.5)                         # leases of the abandoned flows run out
        with FabricClient(port=port) as c:
            assert c.request("FLOWS").startswith("OK n=0")
    finally:
        p.send_signal(signal.SIGTERM)
        try:
            _, err = p.communicate(timeout=20)
        except subprocess.TimeoutExpired:
            p.kill()
            _, err = p.communicate()
    assert p.returncode == 0, err[-3000:]
    assert "Sanitizer" not in err and "runtime error" not in err and "data race" not in err, err[-3000:]
