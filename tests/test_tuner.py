"""The tuner and the benchmark template: rendering, the compile line, result bookkeeping (CPU),
and a real two-configuration tuning run plus the comparison harnesses on a GPU."""
import json
import re
import subprocess
from pathlib import Path

import pytest

from h100_gemm_b200 import build
from h100_gemm_b200.tuner import gemm_tuner as gt

REPO = Path(__file__).resolve().parent.parent


def test_template_renders_for_every_configuration(tmp_path):
    for space in (gt.B200_PARAM_SPACE, gt.REFERENCE_PARAM_SPACE):
        tuner = gt.GemmTuner(output_dir=str(tmp_path), param_space=space)
        configs = tuner.configurations()
        assert len(configs) == len({gt.config_name(c) for c in configs}) > 0
        for c in configs:
            code = tuner.generate_code(c)
            for k, v in c.items():
                assert re.search(rf"static constexpr int {k} = {v};", code)
            assert "{{" not in code
    # the reference's space has the size its tuner walks (gemm_tuner.py:17-24: 5*1*3*1*1*5)
    assert len(gt.GemmTuner(output_dir=str(tmp_path), param_space=gt.REFERENCE_PARAM_SPACE).configurations()) == 75


def test_invalid_cluster_n_is_filtered(tmp_path):
    space = dict(gt.B200_PARAM_SPACE, CLUSTER_N=[1, 2])
    tuner = gt.GemmTuner(output_dir=str(tmp_path), param_space=space)
    assert all(c["CLUSTER_N"] == 1 for c in tuner.configurations())


def test_rendered_template_compiles_for_sm100a(tmp_path):
    build.build_library()
    tuner = gt.GemmTuner(output_dir=str(tmp_path))
    params = dict(CLUSTER_M=2, CLUSTER_N=1, BLOCKM=128, BLOCKN=256, BLOCKK=64, STAGES=6)
    cmd = tuner.compile_command(tmp_path / "t.cu", tmp_path / "t")
    assert "arch=compute_100a,code=sm_100a" in cmd
    assert tuner.compile_configuration(params, tmp_path / "test")
    assert (tmp_path / "test").exists()


def test_bookkeeping_resume_and_failures(tmp_path, monkeypatch):
    space = dict(CLUSTER_M=[1, 2], CLUSTER_N=[1], BLOCKM=[128, 64], BLOCKN=[256], BLOCKK=[64], STAGES=[4])
    calls = []

    def fake(self, params):
        calls.append(gt.config_name(params))
        if params["BLOCKM"] == 64:
            return float("inf"), False          # a configuration with no kernel
        return (0.5 if params["CLUSTER_M"] == 2 else 0.7), True

    monkeypatch.setattr(gt.GemmTuner, "benchmark_configuration", fake)
    tuner = gt.GemmTuner(output_dir=str(tmp_path), param_space=space, shape=(512, 512, 512))
    best, runtime, results = tuner.tune()
    assert best["CLUSTER_M"] == 2 and runtime == 0.5 and len(results) == 4 and len(calls) == 4
    lines = [json.loads(l) for l in (tmp_path / "tuning_results.jsonl").read_text().splitlines()]
    assert len(lines) == 4 and sum(not l["success"] for l in lines) == 2
    assert "static constexpr int CLUSTER_M = 2;" in (tmp_path / "best_matmul_b200.cu").read_text()
    summary = (tmp_path / "tuning_summary.txt").read_text()
    assert "Best runtime: 0.5000 ms" in summary and "Failed configurations" in summary
    # resume: nothing is re-run
    calls.clear()
    best2, runtime2, results2 = gt.GemmTuner(output_dir=str(tmp_path), param_space=space).tune(resume=True)
    assert calls == [] and best2 == best and runtime2 == runtime and len(results2) == 4


def test_latency_line_is_parsed():
    out = "Shape M=5120, N=5120, K=4096\nCorrect!\nAverage latency (ms) is 0.1234\n"
    assert float(gt.LATENCY_RE.search(out).group(1)) == 0.1234


@pytest.mark.gpu
def test_tuner_end_to_end_two_configurations(tmp_path):
    space = dict(CLUSTER_M=[1, 2], CLUSTER_N=[1], BLOCKM=[128], BLOCKN=[128], BLOCKK=[64], STAGES=[4])
    tuner = gt.GemmTuner(output_dir=str(tmp_path), param_space=space, shape=(1024, 1024, 512), timeout=120)
    best, runtime, results = tuner.tune()
    assert best is not None and 0 < runtime < 50 and all(r["success"] for r in results)
    # a configuration without a kernel is a failed run, not a crash of the tuner
    bad = gt.GemmTuner(output_dir=str(tmp_path / "bad"), param_space=dict(space, BLOCKN=[96], CLUSTER_M=[1]),
                       shape=(512, 512, 512), timeout=120)
    best, _, results = bad.tune()
    assert best is None and not results[0]["success"]


@pytest.mark.gpu
def test_blockm_64_of_the_reference_space_runs(tmp_path):
    """BLOCKM = 64, BLOCKN = 128 (gemm_tuner.py:17-24) maps to the few-rows plan: 64 x 128 tiles with
    the operands swapped inside. The template's own check against the SIMT GEMM must pass."""
    space = dict(CLUSTER_M=[1], CLUSTER_N=[1], BLOCKM=[64], BLOCKN=[128], BLOCKK=[64], STAGES=[5])
    tuner = gt.GemmTuner(output_dir=str(tmp_path), param_space=space, shape=(1024, 1024, 512), timeout=120)
    best, runtime, results = tuner.tune()
    assert best is not None and results[0]["success"] and 0 < runtime < 50


@pytest.mark.gpu
def test_comparison_harnesses_run():
    build.build_all()
    subprocess.run(["make", "-C", str(REPO / "h100_gemm_b200" / "bench")], check=True, capture_output=True)
    bin_dir = REPO / "h100_gemm_b200" / "bench" / "bin"
    out = subprocess.run([str(bin_dir / "test"), "M", "1000", "N", "776", "K", "520"], capture_output=True, text=True,
                         timeout=120)
    assert out.returncode == 0 and "Correct!" in out.stdout and gt.LATENCY_RE.search(out.stdout)
    out = subprocess.run([str(bin_dir / "matmul_b200_optimal"), "2048", "4"], capture_output=True, text=True, timeout=120)
    assert out.returncode == 0 and "Verified against cuBLAS" in out.stdout and out.stdout.count("TFLOPS") == 2
    out = subprocess.run([str(bin_dir / "cublas_ref"), "1024", "512", "768", "5"], capture_output=True, text=True,
                         timeout=120)
    assert out.returncode == 0 and "CuBlas_TC" in out.stdout and "CuBlasLt" in out.stdout
    # one process driving every visible GPU through b200_mgemm_* (a single device here or many)
    out = subprocess.run([str(bin_dir / "matmul_b200_multi"), "1024", "768", "520", "3"], capture_output=True, text=True,
                         timeout=300)
    assert out.returncode == 0 and "Correct!" in out.stdout and "P=1" in out.stdout, out.stdout + out.stderr


@pytest.mark.gpu
def test_cutlass_comparator_agrees_bit_for_bit():
    """The CUTLASS Sm100 builder GEMM, this library and the SIMT GEMM give the same bits on
    integer-valued inputs (the harness exits non-zero otherwise). Needs CUTLASS 4.x headers at
    build time; skipped where there are none and no prebuilt binary."""
    binary = REPO / "h100_gemm_b200" / "bench" / "bin" / "cutlass_ref"
    source = REPO / "h100_gemm_b200" / "bench" / "cutlass_ref.cu"
    if not binary.exists() or binary.stat().st_mtime < source.stat().st_mtime:
        made = subprocess.run(["make", "-C", str(REPO / "h100_gemm_b200" / "bench"), "cutlass_ref"], capture_output=True,
                              text=True, timeout=900)
        if made.returncode != 0:
            pytest.skip("CUTLASS headers not available: " + made.stdout[-200:])
    out = subprocess.run([str(binary), "--m=1024", "--n=768", "--k=512", "--iterations=5"], capture_output=True,
                         text=True, timeout=120)
    assert out.returncode == 0, out.stdout + out.stderr
    assert out.stdout.count("Disposition: Passed") == 2 and out.stdout.count("GFLOPS:") == 2
    assert "CUTLASS 0, libb200gemm 0" in out.stdout


@pytest.mark.gpu
def test_vendor_baselines_agree_with_the_kernel():
    import torch

    import h100_gemm_b200 as g
    from h100_gemm_b200 import baselines
    gen = torch.Generator(device="cuda").manual_seed(3)
    a = torch.randint(-5, 5, (1000, 1544), device="cuda", generator=gen).to(torch.bfloat16)
    b = torch.randint(-5, 5, (776, 1544), device="cuda", generator=gen).to(torch.bfloat16)
    ours = g.gemm(a, b)
    assert torch.equal(ours.view(torch.int16), baselines.cublas_gemm(a, b).view(torch.int16))
    assert torch.equal(ours.view(torch.int16), baselines.cublaslt_gemm(a, b).view(torch.int16))
    col = baselines.cublas_gemm(a, b, c_col_major=True)  # [N, M]
    assert torch.equal(ours.t().contiguous().view(torch.int16), col.view(torch.int16))
