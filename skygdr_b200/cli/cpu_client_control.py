"""Send one control command to a flow end-point (or to fabricd) and print the reply.

    python -m skygdr_b200.cli.cpu_client_control --host H --port P [--timeout_s 2] "HIGH|LOW|LOW2..4|SLEEP <us>|STOP|STATUS"

Same interface as src/tools/cpu_client_control.py:9-20.
"""
import argparse
import sys

from skygdr_b200.control.client import send_control


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--host", required=True)
    ap.add_argument("--port", type=int, required=True)
    ap.add_argument("command")
    ap.add_argument("--timeout_s", type=float, default=2.0)
    a = ap.parse_args(argv)
    try:
        print(send_control(a.host, a.port, a.command, a.timeout_s))
    except OSError as exc:
        print(f"control connection failed: {exc}", file=sys.stderr)
        return 1
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
