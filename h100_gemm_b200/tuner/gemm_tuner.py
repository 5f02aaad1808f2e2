"""Grid-search tuner for the sm_100a GEMM template — the counterpart of the reference's
gemm_tuner.py (GemmTuner, gemm_tuner.py:11-164), same flow and same contract with the benchmark
binary: render the Jinja template, compile, run `./test M 5120 N 5120 K 4096`, parse
`Average latency (ms) is <f>` from stdout; a non-zero exit code, a compile error or a timeout
marks the configuration as failed.

What differs from the reference:
  * compile flags: `-gencode arch=compute_100a,code=sm_100a` and the include/library paths of
    this repository (the reference's `-arch=sm_90a` line, gemm_tuner.py:46, targets Hopper);
  * the search space is the one the Blackwell kernel implements (see include/b200_gemm.h); the
    reference's space (gemm_tuner.py:17-24) can still be passed in — configurations without a
    kernel are reported as failed runs, exactly as a failing assert was;
  * results go to ONE append-only JSON-lines file and `--resume` skips what is already there,
    because every GPU minute is budgeted (the reference rewrites a new timestamped JSON after
    every configuration and cannot resume, gemm_tuner.py:128-137);
  * batch mode: `--compile-only DIR` builds one binary per configuration on a machine without a
    GPU, `--run-only DIR` runs prebuilt binaries on the GPU machine;
  * `--shape` may be given several times and `--table FILE` records the best configuration of
    every shape in the text format `b200_gemm_tuning_load` reads (include/b200_gemm.h), so that
    what the search finds is what `cfg == NULL` calls use afterwards. The reference's tuner
    searches one shape and nothing consumes its result (gemm_tuner.py:55,126-145).
"""
from __future__ import annotations

import argparse
import itertools
import json
import re
import subprocess
from datetime import datetime
from pathlib import Path
from typing import Dict, List, Optional, Tuple

from jinja2 import Template

PKG = Path(__file__).resolve().parent.parent
REPO = PKG.parent
DEFAULT_TEMPLATE = PKG / "bench" / "matmul_b200.cu.jinja"

# Decode-like shapes (M <= 128): the few-rows plan's tiles with whole tiles and with stream-K. Pass
# with --space few-rows. SCHED and SWAP_AB are optional template variables (see OPTIONAL_KEYS).
FEW_ROWS_PARAM_SPACE = {
    'CLUSTER_M': [1],
    'CLUSTER_N': [1],
    'BLOCKM': [16, 32, 64, 128],
    'BLOCKN': [128],
    'BLOCKK': [64],
    'STAGES': [6, 8, 9, 11, 12],
    'SCHED': [0, 2],
    'SWAP_AB': [1],
}

# Template variables beyond the reference's six; a parameter dictionary may leave them out (= 0).
OPTIONAL_KEYS = ('SCHED', 'SPLIT_K', 'RASTER', 'GROUP', 'EPILOGUE', 'SWAP_AB')

B200_PARAM_SPACE = {
    'CLUSTER_M': [1, 2],
    'CLUSTER_N': [1],
    'BLOCKM': [128, 256],
    'BLOCKN': [64, 128, 192, 256],
    'BLOCKK': [64],
    'STAGES': [3, 4, 6],
}

# The reference's space (gemm_tuner.py:17-24). BLOCKM = 64 runs as the few-rows plan (64 x 128 tiles,
# operands swapped inside) with CLUSTER_M = 1; larger clusters with it, and STAGES beyond shared
# memory, have no kernel here and come back as failed configurations.
REFERENCE_PARAM_SPACE = {
    'CLUSTER_M': [1, 2, 4, 8, 16],
    'CLUSTER_N': [1],
    'BLOCKM': [64, 128, 256],
    'BLOCKN': [128],
    'BLOCKK': [64],
    'STAGES': [3, 5, 7, 9, 11],
}

TABLE_HEADER = "# batch M N K block_m block_n cluster_m stages sched split_k raster group epilogue swap_ab\n"


def table_line(shape: Tuple[int, int, int], params: Dict[str, int], batch: int = 1) -> str:
    """One tuning-table entry: the template's parameters for `shape` (optional ones default to 0)."""
    m, n, k = shape
    extra = ' '.join(str(params.get(key, 0)) for key in ('SCHED', 'SPLIT_K', 'RASTER', 'GROUP', 'EPILOGUE', 'SWAP_AB'))
    return (f"{batch} {m} {n} {k} {params['BLOCKM']} {params['BLOCKN']} {params['CLUSTER_M']} "
            f"{params['STAGES']} {extra}")


def update_table(path, shape: Tuple[int, int, int], params: Dict[str, int], runtime_ms: Optional[float] = None,
                 batch: int = 1) -> None:
    """Adds or replaces the entry of `shape` in the table file `path` (created if missing)."""
    path = Path(path)
    key = [str(batch)] + [str(v) for v in shape]
    kept = []
    if path.exists():
        for line in path.read_text().splitlines():
            body = line.split('#', 1)[0].split()
            if body[:4] == key:
                continue
            kept.append(line)
    if not kept:
        kept = [TABLE_HEADER.rstrip("\n")]
    note = f"  # {runtime_ms:.4f} ms" if runtime_ms is not None else ""
    kept.append(table_line(shape, params, batch) + note)
    path.write_text("\n".join(kept) + "\n")


LATENCY_RE = re.compile(r"Average latency \(ms\) is ([\d.]+)")


def config_name(params: Dict[str, int]) -> str:
    name = "cm{CLUSTER_M}_cn{CLUSTER_N}_bm{BLOCKM}_bn{BLOCKN}_bk{BLOCKK}_st{STAGES}".format(**params)
    tags = {'SCHED': 's', 'SPLIT_K': 'k', 'RASTER': 'r', 'GROUP': 'g', 'EPILOGUE': 'e', 'SWAP_AB': 'w'}
    return name + ''.join(f"_{tags[key]}{params[key]}" for key in OPTIONAL_KEYS if params.get(key, 0))


class GemmTuner:
    def __init__(self, template_file: str = str(DEFAULT_TEMPLATE), output_dir: str = "tuning_results",
                 param_space: Optional[Dict[str, List[int]]] = None, shape: Tuple[int, int, int] = (5120, 5120, 4096),
                 timeout: int = 30, work_dir: Optional[str] = None):
        self.output_dir = Path(output_dir)
        self.output_dir.mkdir(parents=True, exist_ok=True)
        self.work_dir = Path(work_dir) if work_dir else self.output_dir
        self.work_dir.mkdir(parents=True, exist_ok=True)
        self.param_space = dict(param_space or B200_PARAM_SPACE)
        self.shape = shape
        self.timeout = timeout
        self.results_file = self.output_dir / "tuning_results.jsonl"
        with open(template_file, 'r') as f:
            self.template = Template(f.read())

    # ---- same surface as the reference's class ----
    def generate_code(self, params: Dict[str, int]) -> str:
        """Generate code with given parameters"""
        return self.template.render(**params)

    def is_valid_configuration(self, params: Dict[str, int]) -> bool:
        """Cluster shapes along N are not searched (gemm_tuner.py:74-80)."""
        return params['CLUSTER_N'] <= 1

    def compile_command(self, source: Path, binary: Path) -> List[str]:
        lib_dir = PKG / "lib"
        return ["nvcc", "-gencode", "arch=compute_100a,code=sm_100a", "-std=c++17", str(source), "-o", str(binary),
                f"-I{REPO / 'include'}", f"-L{lib_dir}", "-lb200gemm", "-Xlinker", f"-rpath={lib_dir}"]

    def compile_configuration(self, params: Dict[str, int], binary: Path) -> bool:
        source = binary.with_suffix(".cu")
        source.write_text(self.generate_code(params))
        if binary.exists():
            binary.unlink()
        proc = subprocess.run(self.compile_command(source, binary), capture_output=True, text=True)
        if proc.returncode != 0:
            print(f"Compilation failed for parameters: {params}\n{proc.stderr[-2000:]}")
            return False
        return True

    def run_binary(self, binary: Path, params: Dict[str, int]) -> Tuple[float, bool]:
        m, n, k = self.shape
        try:
            result = subprocess.run([str(binary), 'M', str(m), 'N', str(n), 'K', str(k)], capture_output=True,
                                    text=True, timeout=self.timeout)
        except subprocess.TimeoutExpired:
            print(f"Timeout for parameters: {params}")
            return float('inf'), False
        if result.returncode != 0:
            print(f"Runtime error for parameters: {params}")
            return float('inf'), False
        match = LATENCY_RE.search(result.stdout)
        if match:
            return float(match.group(1)), True
        print(f"Could not parse output for parameters: {params}")
        return float('inf'), False

    def benchmark_configuration(self, params: Dict[str, int]) -> Tuple[float, bool]:
        """Benchmark a single configuration. Returns (runtime, success)"""
        binary = self.work_dir / "test"
        if not self.compile_configuration(params, binary):
            return float('inf'), False
        return self.run_binary(binary, params)

    # ---- search ----
    def configurations(self) -> List[Dict[str, int]]:
        combos = [dict(zip(self.param_space.keys(), values)) for values in itertools.product(*self.param_space.values())]
        return [p for p in combos if self.is_valid_configuration(p)]

    def load_results(self) -> List[Dict]:
        if not self.results_file.exists():
            return []
        return [json.loads(line) for line in self.results_file.read_text().splitlines() if line.strip()]

    def record(self, result: Dict) -> None:
        with open(self.results_file, 'a') as f:
            f.write(json.dumps(result) + "\n")

    def tune(self, resume: bool = False, prebuilt_dir: Optional[str] = None):
        """Run the tuning process and save results"""
        results = self.load_results() if resume else []
        if not resume and self.results_file.exists():
            self.results_file.unlink()
        done = {config_name(r['params']) for r in results}
        best_runtime, best_params = float('inf'), None
        for r in results:
            if r['success'] and r['runtime'] < best_runtime:
                best_runtime, best_params = r['runtime'], r['params']
        configs = self.configurations()
        for i, params in enumerate(configs):
            if config_name(params) in done:
                continue
            print(f"\nTesting configuration {i + 1}/{len(configs)}:\n{params}")
            if prebuilt_dir is not None:
                binary = Path(prebuilt_dir) / config_name(params)
                runtime, success = self.run_binary(binary, params) if binary.exists() else (float('inf'), False)
            else:
                runtime, success = self.benchmark_configuration(params)
            result = {'params': params, 'runtime': runtime if success else None, 'success': success,
                      'shape': list(self.shape), 'timestamp': datetime.now().isoformat()}
            results.append(result)
            self.record(result)
            if success:
                print(f"Runtime: {runtime:.4f} ms")
            if success and runtime < best_runtime:
                best_runtime, best_params = runtime, params
                print(f"New best runtime: {best_runtime:.4f} ms")
                (self.output_dir / 'best_matmul_b200.cu').write_text(self.generate_code(best_params))
            self.save_results(results, best_params, best_runtime)
        return best_params, best_runtime, results

    def compile_all(self, out_dir: str) -> Dict[str, bool]:
        """Batch mode, step 1 (no GPU needed): one binary per configuration in `out_dir`."""
        out = Path(out_dir)
        out.mkdir(parents=True, exist_ok=True)
        return {config_name(p): self.compile_configuration(p, out / config_name(p)) for p in self.configurations()}

    def save_results(self, results: List[Dict], best_params: Optional[Dict[str, int]], best_runtime: float):
        """Summary of all runs so far (the JSON-lines file is the record of truth)."""
        with open(self.output_dir / 'tuning_summary.txt', 'w') as f:
            f.write(f"Tuning updated at: {datetime.now().strftime('%Y%m%d_%H%M%S')}\n")
            f.write(f"Shape: M={self.shape[0]} N={self.shape[1]} K={self.shape[2]}\n")
            f.write(f"Best runtime: {best_runtime:.4f} ms\n")
            if best_params:
                f.write("Best parameters:\n")
                for key, value in best_params.items():
                    f.write(f"{key}: {value}\n")
            f.write("\nAll successful configurations:\n")
            for r in sorted([r for r in results if r['success']], key=lambda x: x['runtime']):
                flops = 2.0 * self.shape[0] * self.shape[1] * self.shape[2]
                f.write(f"\nRuntime: {r['runtime']:.4f} ms ({flops / r['runtime'] / 1e9:.1f} TFLOP/s)\n")
                for k, v in r['params'].items():
                    f.write(f"{k}: {v}\n")
            failed = [config_name(r['params']) for r in results if not r['success']]
            if failed:
                f.write("\nFailed configurations:\n" + "\n".join(failed) + "\n")


def main():
    ap = argparse.ArgumentParser(description=__doc__.splitlines()[0])
    ap.add_argument("--template", default=str(DEFAULT_TEMPLATE))
    ap.add_argument("--output-dir", default="tuning_results")
    ap.add_argument("--space", default="b200", choices=["b200", "reference", "few-rows"])
    ap.add_argument("--shape", type=int, nargs=3, action="append", metavar=("M", "N", "K"),
                    help="shape to tune (default 5120 5120 4096); may be repeated")
    ap.add_argument("--table", metavar="FILE", help="record each shape's best configuration in this tuning table")
    ap.add_argument("--resume", action="store_true")
    ap.add_argument("--compile-only", metavar="DIR")
    ap.add_argument("--run-only", metavar="DIR")
    args = ap.parse_args()
    space = {"b200": B200_PARAM_SPACE, "reference": REFERENCE_PARAM_SPACE, "few-rows": FEW_ROWS_PARAM_SPACE}[args.space]
    shapes = [tuple(sh) for sh in (args.shape or [[5120, 5120, 4096]])]
    if args.compile_only:
        tuner = GemmTuner(args.template, args.output_dir, space, shapes[0])
        built = tuner.compile_all(args.compile_only)
        print(f"compiled {sum(built.values())}/{len(built)} configurations into {args.compile_only}")
        return
    for shape in shapes:
        out_dir = args.output_dir if len(shapes) == 1 else str(Path(args.output_dir) / "x".join(map(str, shape)))
        tuner = GemmTuner(args.template, out_dir, space, shape)
        best_params, best_runtime, _ = tuner.tune(resume=args.resume, prebuilt_dir=args.run_only)
        if best_params:
            print("\nTuning completed!")
            print(f"Best runtime: {best_runtime:.4f} ms")
            print("Best parameters:")
            for key, value in best_params.items():
                print(f"{key}: {value}")
            print(f"\nResults saved in {out_dir}")
            if args.table:
                update_table(args.table, shape, best_params, best_runtime)
                print(f"Tuning table updated: {args.table}")
        else:
            print("\nNo valid configuration found!")


if __name__ == "__main__":
    main()
