"""Trace-shaped KV hand-off: `kv_nvlink_transfer --trace` under the reference's program name
(llm_problem_analysis/kv_nvlink_transfer_trace.cu)."""
import sys

from .kv_nvlink_transfer import main as _main


def main(argv=None) -> int:
    return _main(["--trace"] + list(sys.argv[1:] if argv is None else argv))


if __name__ == "__main__":
    raise SystemExit(main())
