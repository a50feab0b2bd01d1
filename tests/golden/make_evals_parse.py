"""Writes tests/golden/evals_parsed_by_reference.json: what the reference's own plotting script
(evals/plot_results.py, parse_h100 / parse_sgemm / parse_scan, lines 18-108) extracts from the sample outputs of
this repository's evaluation programs under tests/golden/evals_output_b200/ (captured on a B200:
prism_b200/evals/build/sgemm_sweep, scan_bench 30, bf16_bench).

    PRISM_REFERENCE=/path/to/prism python tests/golden/make_evals_parse.py

The script is imported unmodified from the checkout; matplotlib, which it imports for its plots and which need not
be installed, is replaced by an empty stand-in because only the parsing functions are called.
"""
import importlib.util
import json
import os
import sys
import types
from pathlib import Path

HERE = Path(__file__).resolve().parent
SAMPLES = HERE / "evals_output_b200"


def load_reference_parser(reference_root):
    """The reference's evals/plot_results.py as a module, with stand-ins for the matplotlib modules it imports."""
    path = Path(reference_root) / "evals" / "plot_results.py"
    if not path.is_file():
        return None
    saved = {k: sys.modules.get(k) for k in ("matplotlib", "matplotlib.pyplot", "matplotlib.ticker")}
    try:
        if importlib.util.find_spec("matplotlib") is None:
            pkg = types.ModuleType("matplotlib")
            pkg.pyplot = types.ModuleType("matplotlib.pyplot")
            pkg.ticker = types.ModuleType("matplotlib.ticker")
            sys.modules.update({"matplotlib": pkg, "matplotlib.pyplot": pkg.pyplot, "matplotlib.ticker": pkg.ticker})
        spec = importlib.util.spec_from_file_location("prism_reference_plot_results", path)
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
        return mod
    finally:
        for k, v in saved.items():
            if v is None:
                sys.modules.pop(k, None)
            else:
                sys.modules[k] = v


def parse_samples(mod):
    def lines(name):
        return (SAMPLES / name).read_text().splitlines(keepends=True)
    return {
        "bf16": [list(r) for r in mod.parse_h100(lines("bf16_bench.txt"))],
        "sgemm": {k: [list(r) for r in v] for k, v in mod.parse_sgemm(lines("sgemm_sweep.txt")).items()},
        "scan": [list(r) for r in mod.parse_scan(lines("scan_bench.txt"))],
    }


def main():
    root = os.environ.get("PRISM_REFERENCE", str(HERE.parent.parent.parent / "reference"))
    mod = load_reference_parser(root)
    if mod is None:
        sys.exit(f"no evals/plot_results.py under {root}; set PRISM_REFERENCE")
    out = HERE / "evals_parsed_by_reference.json"
    out.write_text(json.dumps(parse_samples(mod)) + "\n")
    print("wrote", out)


if __name__ == "__main__":
    main()
