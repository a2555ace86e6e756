"""The CPU arm of bench.py: it uses every host core even when a launcher exported OMP_NUM_THREADS=1, says which sample it
sorts, and loads nothing of the product; its corpus generator (under oracle/) makes the same symbols as the product's."""
import json
import os
import subprocess
import sys

import numpy as np

from conftest import ROOT


def test_oracle_corpus_equals_the_products(oracle):
    sys.path.insert(0, ROOT)
    import bench
    from cascade_b200 import api
    assert np.array_equal(bench.zipf_cdf(), api.zipf_cdf())
    cpu = bench.CpuSide()
    for n, mean_doc, seed in ((100000, 1024, 0), (50000, 3, 7)):
        a = cpu.corpus(n, mean_doc, seed)
        b = api.gen_corpus_host(n, seed, mean_doc)
        assert np.array_equal(a[:n], b[:n])


def test_reference_arm_under_a_launcher_that_pins_one_thread():
    env = dict(os.environ, OMP_NUM_THREADS="1", RANK="0", WORLD_SIZE="2", LOCAL_RANK="0")
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--gpus", "2", "--steps", "1", "--warmup", "0",
                          "--ref-sample", "200000"], env=env, capture_output=True, text=True, timeout=300)
    assert out.returncode == 0, out.stderr
    line = json.loads(out.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference" and line["n_gpus"] == 2 and line["gpu_launches"] == 0
    assert line["config"]["reference_sample_tokens"] == 200000 and "sample" in line["config"]["workload"]
    assert line["cpu_baseline"]["cores"] == len(os.sched_getaffinity(0))
    assert line["e2e"]["h2d_bytes_per_step"] == 0 and line["e2e"]["value"] == line["value"]
    # the other ranks of a multi-rank launch print nothing and exit 0
    env["RANK"] = "1"
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--gpus", "2", "--steps", "1", "--warmup", "0",
                          "--ref-sample", "200000"], env=env, capture_output=True, text=True, timeout=300)
    assert out.returncode == 0 and out.stdout.strip() == ""


def test_reference_arm_loads_no_product_library():
    code = ("import sys, bench; sys.argv=['bench.py','--impl','reference','--steps','1','--warmup','0','--ref-sample','50000']; bench.main(); "
            "maps=open('/proc/self/maps').read(); assert 'libcascade_b200' not in maps and 'torch' not in maps, 'product or torch library loaded'")
    out = subprocess.run([sys.executable, "-c", code], cwd=ROOT, capture_output=True, text=True, timeout=300)
    assert out.returncode == 0, out.stderr
