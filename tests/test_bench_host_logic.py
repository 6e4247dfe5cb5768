"""Host logic of bench.py that needs no GPU: what every rank of a multi-GPU run must agree on, and the CPU arm's line."""
import json
import os
import subprocess
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
import bench  # noqa: E402


def test_every_rank_gets_the_same_lengths_in_its_own_order():
    """Weak scaling means the same work per GPU: the step time is a maximum over ranks and followed the heaviest draw
    when every rank drew its own lengths."""
    w = bench.WORKLOADS["glm4_9b_batched_decode"]
    base = np.sort(bench.draw_n_past(w, 0))
    for rank in range(1, 8):
        mine = bench.draw_n_past(w, rank)
        assert np.array_equal(np.sort(mine), base)
        assert not np.array_equal(mine, bench.draw_n_past(w, 0))
    assert base.min() >= w["n_past"][0] and base.max() <= w["n_past"][1]


def test_split_kv_rotation_count_is_the_same_on_every_rank():
    """The ranks capture graphs of `rotation` steps and replay them the same number of times: a count that depends on the
    rank's own slice (the last rank's is shorter) makes them run different numbers of exchange steps."""
    from chatglm_cpp_b200 import sharding
    w = bench.WORKLOADS["glm4_9b_long_131072"]
    P = w["n_past"][0]
    for world in (1, 2, 4, 8):
        n_rot = bench.split_kv_rotation(P, world, w["G"], w["D"])
        slices = [sharding.split_kv(P, 0, world, r) for r in range(world)]
        assert sum(s.n_local for s in slices) == P
        per_rank = {max(2, int(np.ceil(4 * 126e6 / (4 * w["G"] * w["D"] * (s.n_local + int(s.owns_new)))))) for s in slices}
        # the per-rank formula is what used to be there: it disagrees between ranks at 4 and 8 ranks
        assert len(per_rank) > 1 or world <= 2
        assert n_rot * 4 * w["G"] * w["D"] * sharding.slice_capacity(P, 0, world) >= 4 * 126e6


def test_reference_arm_prints_one_line_with_the_contract_keys():
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--steps", "1", "--warmup", "1",
                          "--workload", "glm3_6b_decode_512"], capture_output=True, text=True, cwd=ROOT, timeout=600)
    assert out.returncode == 0, out.stderr[-500:]
    line = json.loads(out.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference" and line["unit"] == "tokens/s" and line["higher_is_better"] is True
    assert line["cpu_baseline"]["kind"] == "port" and line["cpu_baseline"]["cores"] >= 1
    assert line["e2e"]["h2d_bytes_per_step"] == 0 and line["e2e"]["d2h_bytes_per_step"] == 0
    assert line["config"]["workload"] == "glm3_6b_decode_512" and line["value"] > 0
    assert "executes" in line["cpu_baseline"]["sample"]


def test_workload_table_is_well_formed_and_the_default_run_names_exist():
    """A misspelt workload name or a missing key would only show on a GPU box: every entry carries what its measurement
    reads, the names the default run asks for exist, and every workload fits the device memory it is documented for."""
    import inspect
    import re
    common = {"H", "G", "D", "M", "layers", "seqs", "n_past", "rope", "theta", "mask", "interleaved", "seed"}
    kinds = ("prefill", "qkv_linear", "attention_block", "split_kv")
    for name, w in bench.WORKLOADS.items():
        assert common <= set(w), (name, common - set(w))
        assert sum(1 for k in kinds if w.get(k)) <= 1, name
        assert w["H"] % w["G"] == 0 and w["n_past"][0] <= w["n_past"][1] < w["M"], name
        slots = w["layers"] * w["seqs"]
        cache_bytes = slots * 2 * w["G"] * w["M"] * w["D"] * 2
        assert cache_bytes <= 60e9, (name, cache_bytes)             # a third of a B200's 180 GB at most
        if w.get("attention_block") or w.get("qkv_linear"):
            hidden = w.get("attention_block") or w["qkv_linear"]
            assert hidden % 64 == 0 and ((w["H"] + 2 * w["G"]) * w["D"]) % 32 == 0, name
            assert w["layers"] * (w["H"] + 2 * w["G"]) * w["D"] * hidden * 2 > 126e6, name   # weights in rotation exceed L2
    assert bench.HEADLINE in bench.WORKLOADS
    asked = set(re.findall(r'"(glm[0-9a-z_]+)"', inspect.getsource(bench.run_default)))
    assert asked and asked <= set(bench.WORKLOADS), asked - set(bench.WORKLOADS)
