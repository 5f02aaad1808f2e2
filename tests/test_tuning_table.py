"""The tuning table behind cfg == NULL: lookup rules, file format, and the tuner's writer.
Pure host logic of libb200gemm.so — no GPU, no compute call."""
import os
import subprocess
import sys
from pathlib import Path

import pytest

import h100_gemm_b200 as g
from h100_gemm_b200.tuner import gemm_tuner

REPO = Path(__file__).resolve().parent.parent
MEASURED = REPO / "h100_gemm_b200" / "tuner" / "b200_measured.table"


@pytest.fixture(autouse=True)
def empty_table():
    g.tuning_clear()
    yield
    g.tuning_clear()


def tiles(cfg):
    return (cfg.block_m, cfg.block_n, cfg.cluster_m)


def test_empty_table_gives_the_heuristic():
    assert g.tuning_size() == 0
    for shape in [(8192, 8192, 8192), (1024, 1024, 1024), (16, 28672, 8192), (300, 200, 77)]:
        d, h = g.default_config(1, *shape), g.heuristic_config(1, *shape)
        assert (tiles(d), d.sched, d.epilogue) == (tiles(h), h.sched, h.epilogue)


def test_exact_shape_wins_and_replaces():
    cfg = g.GemmConfig(block_m=128, block_n=128, cluster_m=1, stages=4)
    g.tuning_add(4096, 4096, 4096, cfg)
    got = g.default_config(1, 4096, 4096, 4096)
    assert tiles(got) == (128, 128, 1) and got.stages == 4
    g.tuning_add(4096, 4096, 4096, g.GemmConfig(block_m=256, block_n=128, cluster_m=1, stages=3))
    assert g.tuning_size() == 1
    assert tiles(g.default_config(1, 4096, 4096, 4096)) == (256, 128, 1)


def test_class_match_takes_the_nearest_entry_of_the_same_class():
    # class of 3000 is (12, 12, 12): 2049..4096
    g.tuning_add(2304, 2304, 2304, g.GemmConfig(block_m=256, block_n=256, cluster_m=1, stages=3))
    g.tuning_add(4096, 4096, 4096, g.GemmConfig(block_m=128, block_n=192, cluster_m=1, stages=3))
    g.tuning_add(8192, 8192, 8192, g.GemmConfig(block_m=256, block_n=128, cluster_m=1, stages=3))
    assert tiles(g.default_config(1, 3800, 3800, 3800)) == (128, 192, 1)
    assert tiles(g.default_config(1, 2500, 2500, 2500)) == (256, 256, 1)
    # another class: table silent, heuristic answers
    assert tiles(g.default_config(1, 1024, 1024, 1024)) == tiles(g.heuristic_config(1, 1024, 1024, 1024))
    # batched and plain problems never share entries
    assert tiles(g.default_config(4, 4096, 4096, 4096)) == tiles(g.heuristic_config(4, 4096, 4096, 4096))


def test_a_neighbour_that_quantises_badly_on_this_shape_is_not_taken():
    # 2048^3 measured best with 128 x 256 single-CTA tiles (128 tiles on 148 SMs). On 1536^3 the
    # same tiles would be 72, on half the machine: the heuristic's own choice stands there.
    g.tuning_add(2048, 2048, 2048, g.GemmConfig(block_m=128, block_n=256, cluster_m=1, stages=4))
    assert tiles(g.default_config(1, 2048, 2048, 2048)) == (128, 256, 1)
    assert tiles(g.default_config(1, 1536, 1536, 1536)) == tiles(g.heuristic_config(1, 1536, 1536, 1536))
    assert tiles(g.default_config(1, 1920, 2048, 2048)) == (128, 256, 1)   # 120 tiles: still one full wave


def test_stages_that_do_not_fit_a_neighbouring_shape_fall_back_to_as_many_as_fit():
    # 12 stages of (72 rows of A + 64 rows of B) fit in shared memory; with the 128 rows of M = 128 only 9 do
    few = g.GemmConfig(block_m=128, block_n=64, cluster_m=1, stages=12, sched=2, epilogue=2)
    g.tuning_add(72, 8192, 8192, few)
    assert g.default_config(1, 72, 8192, 8192).stages == 12
    near = g.default_config(1, 128, 8192, 8192)
    assert tiles(near) == (128, 64, 1) and 2 <= near.stages < 12


def test_entries_without_a_kernel_are_refused():
    with pytest.raises(g.GemmError):
        g.tuning_add(4096, 4096, 4096, g.GemmConfig(block_m=96, block_n=128, cluster_m=1))
    with pytest.raises(g.GemmError):
        g.tuning_add(4096, 4096, 4096, g.GemmConfig(block_m=128, block_n=96, cluster_m=1))
    with pytest.raises(g.GemmError):
        g.tuning_add(4096, 4096, 4096, g.GemmConfig(block_m=128, block_n=128, cluster_m=1, c_col_major=1))
    with pytest.raises(g.GemmError):
        g.tuning_add(0, 4096, 4096, g.GemmConfig())
    assert g.tuning_size() == 0


def test_load_file_roundtrip_and_errors(tmp_path):
    n = len([l for l in MEASURED.read_text().splitlines() if l.split('#', 1)[0].strip()])
    assert n >= 4 and g.tuning_load(MEASURED) == n
    assert g.tuning_size() == n
    assert tiles(g.default_config(1, 2048, 2048, 2048)) == (128, 256, 1)
    assert g.default_config(1, 2048, 2048, 2048).stages == 4
    assert tiles(g.default_config(1, 8192, 8192, 8192)) == (256, 256, 2)
    few = g.default_config(1, 16, 28672, 8192)
    assert (few.block_m, few.sched, few.swap_ab, few.stages) == (16, 2, 1, 9)
    bad = tmp_path / "bad.table"
    bad.write_text("1 1024 1024 1024 128 128 1 4 0 0 0 0 0\n1 512 512 512 128 128 1\n")
    with pytest.raises(g.GemmError):
        g.tuning_load(bad)
    assert g.tuning_size() == n                      # nothing of a bad file is kept
    nokernel = tmp_path / "nokernel.table"
    nokernel.write_text("1 1024 1024 1024 96 128 1 4 0 0 0 0 0\n")
    with pytest.raises(g.GemmError):
        g.tuning_load(nokernel)
    with pytest.raises(g.GemmError):
        g.tuning_load(tmp_path / "missing.table")
    empty = tmp_path / "empty.table"
    empty.write_text("# nothing here\n\n")
    assert g.tuning_load(empty) == 0


def test_tuner_writes_what_the_library_reads(tmp_path):
    table = tmp_path / "t.table"
    p1 = {'CLUSTER_M': 2, 'CLUSTER_N': 1, 'BLOCKM': 128, 'BLOCKN': 256, 'BLOCKK': 64, 'STAGES': 6}
    p2 = {'CLUSTER_M': 1, 'CLUSTER_N': 1, 'BLOCKM': 256, 'BLOCKN': 128, 'BLOCKK': 64, 'STAGES': 4}
    gemm_tuner.update_table(table, (5120, 5120, 4096), p1, 0.1256)
    gemm_tuner.update_table(table, (1024, 2048, 512), p2)
    gemm_tuner.update_table(table, (5120, 5120, 4096), p2, 0.1)      # replaces the first entry
    assert g.tuning_load(table) == 2
    assert tiles(g.default_config(1, 5120, 5120, 4096)) == (256, 128, 1)
    assert g.default_config(1, 1024, 2048, 512).stages == 4
    text = table.read_text()
    assert text.startswith("# batch M N K") and text.count("5120 5120 4096") == 1


def test_shipped_table_is_loaded_when_no_environment_variable_is_set():
    """cfg == NULL sees the measured entries without any set-up by the caller; an empty value of
    the variable switches the default table off."""
    entries = [line.split('#', 1)[0].split() for line in MEASURED.read_text().splitlines()]
    entries = [[int(x) for x in e] for e in entries if e]
    assert entries
    code = ("import h100_gemm_b200 as g\n"
            f"for e in {entries!r}:\n"
            "    c = g.default_config(e[0], e[1], e[2], e[3])\n"
            "    print(c.block_m, c.block_n, c.cluster_m, c.sched, c.epilogue, c.swap_ab, g.tuning_size())\n")
    env = {k: v for k, v in os.environ.items() if k != "B200_GEMM_TUNING_TABLE"}
    out = subprocess.run([sys.executable, "-c", code], cwd=REPO, env=env, capture_output=True, text=True, check=True)
    rows = [[int(x) for x in line.split()] for line in out.stdout.splitlines()]
    assert len(rows) == len(entries)
    for e, r in zip(entries, rows):
        swap = e[13] if len(e) > 13 else 0
        assert r == [e[4], e[5], e[6], e[8], e[12], swap, len(entries)]
    off = subprocess.run([sys.executable, "-c", "import h100_gemm_b200 as g; g.default_config(1, 2048, 2048, 2048); print(g.tuning_size())"],
                         cwd=REPO, env=dict(env, B200_GEMM_TUNING_TABLE=""), capture_output=True, text=True, check=True)
    assert off.stdout.split() == ["0"]


def test_heuristic_counts_waves_over_the_sms_it_is_given():
    from h100_gemm_b200 import api
    # few rows, 140 tiles of 128 columns: one wave of whole tiles on 148 SMs, stream-K on 132
    assert api.heuristic_config_for_sms(1, 16, 128 * 140, 4096, 148).sched == 0
    assert api.heuristic_config_for_sms(1, 16, 128 * 140, 4096, 132).sched == 2
    # 4096^3: 128 pair tiles of 512 x 256 are two waves on 74 pairs; with 128 pairs they are one,
    # and so are the 256 tiles of 256 x 256 — the smaller tile then costs nothing extra
    # 65..128 rows: whole 224-column tiles while they fit one wave of the device's SMs, 256-column
    # ones (from 97 rows) when only those fit, stream-K beyond — and for a narrow C with a long K
    h = api.heuristic_config_for_sms
    assert (h(1, 128, 28672, 8192, 148).block_n, h(1, 128, 28672, 8192, 148).sched) == (224, 0)
    assert (h(1, 128, 28672, 8192, 120).block_n, h(1, 128, 28672, 8192, 120).sched) == (256, 0)
    assert (h(1, 128, 28672, 8192, 100).block_n, h(1, 128, 28672, 8192, 100).sched) == (128, 2)
    assert (h(1, 80, 28672, 8192, 120).block_n, h(1, 80, 28672, 8192, 120).sched) == (128, 2)
    assert (h(1, 128, 512, 65536, 148).block_n, h(1, 128, 512, 65536, 148).sched) == (128, 2)
    assert api.heuristic_config_for_sms(1, 4096, 4096, 4096, 148).block_m == 256
    assert api.heuristic_config_for_sms(1, 4096, 4096, 4096, 512).block_m == 128
    with pytest.raises(api.GemmError):
        api.heuristic_config_for_sms(1, 16, 128, 128, 0)


def test_environment_variable_loads_a_table_before_the_first_lookup():
    code = ("import h100_gemm_b200 as g; c = g.default_config(1, 2048, 2048, 2048); "
            "print(g.tuning_size(), c.block_m, c.block_n, c.cluster_m, c.stages)")
    env = dict(os.environ, B200_GEMM_TUNING_TABLE=str(MEASURED))
    out = subprocess.run([sys.executable, "-c", code], cwd=REPO, env=env, capture_output=True, text=True, check=True)
    assert out.stdout.split()[1:] == ["128", "256", "1", "4"] and int(out.stdout.split()[0]) >= 4


@pytest.mark.gpu
def test_table_entry_is_what_a_call_without_cfg_runs():
    """cfg=None with a table entry gives the bits of the same call with that cfg spelled out, and
    both agree with the CPU oracle."""
    import torch
    from oracle import oracle
    M, N, K = 768, 1024, 512
    gen = torch.Generator(device="cuda").manual_seed(11)
    a = torch.randint(-5, 5, (M, K), device="cuda", generator=gen).to(torch.bfloat16)
    b = torch.randint(-5, 5, (N, K), device="cuda", generator=gen).to(torch.bfloat16)
    entry = g.GemmConfig(block_m=128, block_n=192, cluster_m=1, stages=3)
    assert tiles(g.heuristic_config(1, M, N, K)) != tiles(entry)
    g.tuning_add(M, N, K, entry)
    assert tiles(g.default_config(1, M, N, K)) == tiles(entry)
    via_table = g.gemm(a, b)
    spelled = g.gemm(a, b, cfg=entry)
    torch.cuda.synchronize()
    assert torch.equal(via_table.view(torch.int16), spelled.view(torch.int16))
    want = oracle.cpu_gemm(a.cpu().view(torch.int16).numpy().view("uint16"),
                                b.cpu().view(torch.int16).numpy().view("uint16"))
    assert (via_table.cpu().view(torch.int16).numpy().view("uint16") == want).all()
    assert g.device_status()[0] == 0
