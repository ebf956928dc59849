"""``python -m skygdr_b200``: what is in the package and how to start it."""
import importlib
import pkgutil
import sys


def main() -> int:
    import skygdr_b200.cli as cli

    print("skygdr_b200: control plane (skygdr_b200.control), kernels (skygdr_b200.ops), models, parallel engines.\n")
    print("Build:      python -m skygdr_b200.build all")
    print("Daemon:     skygdr_b200/bin/fabricd --port 7070 [--policy target_track] [--link NAME=GBPS] [--unix PATH]")
    print("Config 1:   python -m skygdr_b200.control.config1 [--live | --processes]")
    print("Benchmark:  python bench.py --gpus 1   (torch.distributed.run for more GPUs)\n")
    print("Programs and tools (python -m skygdr_b200.cli.<name> --help):")
    for m in sorted(pkgutil.iter_modules(cli.__path__), key=lambda m: m.name):
        if m.name in ("common",):
            continue
        doc = (importlib.import_module(f"skygdr_b200.cli.{m.name}").__doc__ or "").strip().splitlines()
        print(f"  {m.name:<34}{doc[0] if doc else ''}")
    return 0


if __name__ == "__main__":
    sys.exit(main())
