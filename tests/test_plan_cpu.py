"""The query planner (host code): plans, strides and refusals by the reference's rules (src/Query_Engine.cu:822-1006), and
the `query plan` command line."""
import ctypes
import os
import subprocess

import numpy as np

from conftest import ROOT

GB = 10**9


def _plan(n, dev, host, stride=0, tier=0):
    from cascade_b200._lib import QueryPlacement, lib
    pl = QueryPlacement()
    assert lib().csa_query_plan(n, dev, host, stride, tier, ctypes.byref(pl)) == 0
    return pl


def test_plans_in_order_with_margins_and_the_finest_stride_that_fits():
    n = 2 * 10**9                                   # text 4 GB, suffix array 10 GB, table of stride 32: 1 GB
    a = _plan(n, 180 * GB, 1000 * GB)
    assert chr(a.plan) == "A" and a.stride == 32 and a.key_words == 2 and a.table_bytes == (n + 31) // 32 * 16
    assert a.device_margin == 180 * GB // 16 and a.host_bytes == 0 and a.device_bytes < 17 * GB
    # too little device memory for the suffix array: it goes to pinned host memory
    b = _plan(n, 10 * GB, 1000 * GB)
    assert chr(b.plan) == "B" and b.stride == 32 and b.host_bytes >= 5 * n and b.device_bytes < 9 * GB
    assert b.device_margin == 2**30                 # a sixteenth of 10 GB is below the least margin
    # the table takes what is left: a coarser stride where the finest does not fit
    tight = _plan(n, int(15.9 * GB), 1000 * GB)
    assert chr(tight.plan) == "A" and tight.stride > 32 and tight.device_bytes + tight.device_margin <= int(15.9 * GB)
    # named tiers are kept; a stride that is given is kept
    assert chr(_plan(n, 180 * GB, 1000 * GB, tier=2).plan) == "B"
    assert _plan(n, 180 * GB, 1000 * GB, stride=1024).stride == 1024
    # nothing fits: no plan, and the reason names both plans
    none = _plan(n, 3 * GB, 1000 * GB)
    assert none.plan == 0 and b"A takes" in none.why and b"B takes" in none.why
    # the pinned tier needs the host's budget
    nohost = _plan(n, 10 * GB, 5 * GB)
    assert nohost.plan == 0 and b"pinned host memory" in nohost.why


def test_query_plan_command_line(tmp_path):
    tmp = str(tmp_path)
    n = 5000
    rng = np.random.default_rng(1)
    rng.integers(0, 100, n).astype("<u2").tofile(os.path.join(tmp, "text.u16"))
    np.zeros(5 * n, np.uint8).tofile(os.path.join(tmp, "text.sa40"))
    tool = os.path.join(ROOT, "cascade_b200", "bin", "sa_convert")
    # index.meta by hand: the planner reads only n
    with open(os.path.join(tmp, "index.meta"), "w") as f:
        f.write(f"format=gpu_saca_query_index\nformat_version=1\nn={n}\nsym_bytes=2\nsa_width=5\nsa_order=numeric_eot_smallest\ntext=text.u16\n"
                f"sa_part_c=1\nsa_part_0=text.sa40\nsa_part_off_0=0\nsep=65535\nsa_source=test\ncreated_utc=now\n")
    q = os.path.join(ROOT, "cascade_b200", "bin", "query")
    r = subprocess.run([q, "plan", "--index", tmp, "--device-budget", str(8 * GB), "--host-budget", str(64 * GB)], capture_output=True, text=True)
    kv = dict(line.split("=", 1) for line in r.stdout.strip().splitlines())
    assert r.returncode == 0 and kv["plan"] == "A" and kv["stride"] == "32" and kv["sa_res"] == "device" and kv["lanes"] == "3", r.stdout + r.stderr
    r = subprocess.run([q, "plan", "--index", tmp, "--device-budget", str(8 * GB), "--host-budget", str(64 * GB), "--sa-res", "pinned", "--stride", "64"],
                       capture_output=True, text=True)
    kv = dict(line.split("=", 1) for line in r.stdout.strip().splitlines())
    assert r.returncode == 0 and kv["plan"] == "B" and kv["stride"] == "64" and kv["sa_res"] == "pinned"
    # the reference's host-search tiers and comma lists are refused with a reason, not ignored
    for extra in (["--sa-res", "mapped"], ["--text-res", "pageable"], ["--stride", "32,64"]):
        r = subprocess.run([q, "plan", "--index", tmp, "--device-budget", str(8 * GB), "--host-budget", str(64 * GB)] + extra, capture_output=True, text=True)
        assert r.returncode == 1 and "plan=none" in r.stdout and "why=" in r.stdout, extra
    assert os.path.exists(tool)
