"""The command lines of the drop-in surface. CPU part: `query gen` / `query info` and the file formats; GPU part: `cascade`
builds a file byte-equal to the oracle's array and `query find` reproduces the oracle's intervals and counts hash."""
import os
import struct
import subprocess

import numpy as np
import pytest

from conftest import ROOT

BIN = os.path.join(ROOT, "cascade_b200", "bin")


def _write_index(tmp, T, sa40=None):
    T.astype("<u2").tofile(os.path.join(tmp, "text.u16"))
    if sa40 is not None:
        sa40[:5 * len(T)].tofile(os.path.join(tmp, "text.sa40"))
    with open(os.path.join(tmp, "index.meta"), "w") as f:
        f.write(f"format=gpu_saca_query_index\nformat_version=1\nn={len(T)}\nsym_bytes=2\nsa_width=5\nsa_order=numeric_eot_smallest\n"
                f"text=text.u16\nsa_part_c=1\nsa_part_0=text.sa40\nsa_part_off_0=0\nsep=65535\nsa_source=test\ncreated_utc=2026-01-01T00:00:00Z\n")


def _read_qry(path):
    b = open(path, "rb").read()
    magic, version, sym_bytes, q_c, sym_c, mn, mx, seed, _ = struct.unpack("<8sIIQQQQQQ", b[:64])
    assert magic == b"GSAQRY01" and version == 1 and sym_bytes == 2
    off = np.frombuffer(b, dtype="<u8", count=q_c + 1, offset=64)
    sym = np.frombuffer(b, dtype="<u2", count=sym_c, offset=64 + 8 * (q_c + 1))
    return off, sym, (mn, mx, seed)


def _kv(out):
    return dict(line.split("=", 1) for line in out.strip().splitlines() if "=" in line)


def test_query_gen_and_info_without_a_gpu(tmp_path):
    from cascade_b200 import api
    tmp = str(tmp_path)
    T = api.gen_corpus_host(50000, 1, 128)[:50000]
    _write_index(tmp, T)
    for kind, seed in (("substring", 1), ("random", 2)):
        out = os.path.join(tmp, kind + ".qry")
        r = subprocess.run([os.path.join(BIN, "query"), "gen", "--index", tmp, "--out", out, "--kind", kind, "--q", "300", "--len",
                            "1,2,3,4,5,6,7,8,9,10,11,12,13,14,15,16", "--seed", str(seed), "--vocab", "50257"], capture_output=True, text=True)
        assert r.returncode == 0, r.stderr
        off, sym, (mn, mx, sd) = _read_qry(out)
        woff, wsym = api.gen_queries(kind, T if kind == "substring" else None, 50000 if kind == "substring" else 0, 300, seed=seed)
        assert np.array_equal(off, woff) and np.array_equal(sym, wsym) and sd == seed and 1 <= mn <= mx <= 16
    # mutated: the substrings of the same seed with exactly one symbol replaced; unigram: every symbol of the vocabulary once
    out = os.path.join(tmp, "mutated.qry")
    r = subprocess.run([os.path.join(BIN, "query"), "gen", "--index", tmp, "--out", out, "--kind", "mutated", "--q", "300", "--len",
                        "1,2,3,4,5,6,7,8,9,10,11,12,13,14,15,16", "--seed", "1", "--vocab", "50257"], capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    off, sym, _ = _read_qry(out)
    woff, wsym = api.gen_queries("substring", T, 50000, 300, seed=1)
    assert np.array_equal(off, woff)
    changed = np.add.reduceat((sym[:int(off[-1])] != wsym[:int(off[-1])]).astype(np.int64), off[:-1].astype(np.int64))
    diff = sym[:int(off[-1])] != wsym[:int(off[-1])]
    assert np.all(changed == 1) and sym[:int(off[-1])][diff].max() < 50257
    out = os.path.join(tmp, "unigram.qry")
    r = subprocess.run([os.path.join(BIN, "query"), "gen", "--index", tmp, "--out", out, "--kind", "unigram", "--vocab", "300"], capture_output=True, text=True)
    assert r.returncode == 0 and _kv(r.stdout)["q"] == "300", r.stderr
    off, sym, _ = _read_qry(out)
    assert np.array_equal(off, np.arange(301)) and np.array_equal(sym[:300], np.arange(300))
    r = subprocess.run([os.path.join(BIN, "query"), "gen", "--index", tmp, "--out", out, "--kind", "nonsense"], capture_output=True, text=True)
    assert r.returncode != 0 and "substring, mutated, random, unigram" in r.stderr
    r = subprocess.run([os.path.join(BIN, "query"), "info", "--index", tmp], capture_output=True, text=True)
    assert r.returncode == 0 and _kv(r.stdout)["n"] == "50000"
    r = subprocess.run([os.path.join(BIN, "query"), "bogus"], capture_output=True, text=True)
    assert r.returncode != 0 and "Usage" in r.stderr
    r = subprocess.run([os.path.join(BIN, "cascade")], capture_output=True, text=True)
    assert r.returncode != 0 and "Usage: cascade <text-file> <suffix-array-file>" in r.stderr


def test_sa_convert_modes_without_a_gpu(tmp_path, oracle):
    """`sa_convert` (host code): 64-bit entries into 5-byte parts with range, permutation and order checks; metadata for a
    finished 5-byte array; widening back. A damaged array is refused."""
    from cascade_b200 import api
    from conftest import sa40_to_u64
    tmp = str(tmp_path)
    n = 20011
    T = api.gen_corpus_host(n, 3, 64)[:n]
    T.astype("<u2").tofile(os.path.join(tmp, "text.u16"))
    sa40 = oracle.build_sa40(T)[:5 * n]
    sa64 = sa40_to_u64(sa40, n).astype("<u8")
    sa64.tofile(os.path.join(tmp, "sa.u64"))
    tool = os.path.join(BIN, "sa_convert")
    common = ["--text", os.path.join(tmp, "text.u16"), "--sym-bytes", "2"]

    # conversion into one part, every adjacent pair checked
    idx = os.path.join(tmp, "idx")
    r = subprocess.run([tool, "--in", os.path.join(tmp, "sa.u64"), "--index-dir", idx, "--spot", str(n), "--sep", "65535"] + common, capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    assert np.array_equal(np.fromfile(os.path.join(idx, "sa.u40"), dtype=np.uint8), sa40)
    r = subprocess.run([os.path.join(BIN, "query"), "info", "--index", idx], capture_output=True, text=True)
    kv = _kv(r.stdout)
    assert r.returncode == 0 and kv["n"] == str(n) and kv["sa_part_c"] == "1" and kv["sep"] == "65535"

    # conversion into three parts cut at 4096-byte pages
    dirs = [os.path.join(tmp, f"d{i}") for i in range(3)]
    idx3 = os.path.join(tmp, "idx3")
    r = subprocess.run([tool, "--in", os.path.join(tmp, "sa.u64"), "--index-dir", idx3, "--parts", "3", "--part-dirs", ":".join(dirs)] + common,
                       capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    parts = [np.fromfile(os.path.join(d, f"sa.u40.part{i}"), dtype=np.uint8) for i, d in enumerate(dirs)]
    assert np.array_equal(np.concatenate(parts), sa40)
    meta = _kv(open(os.path.join(idx3, "index.meta")).read())
    offs = [int(meta[f"sa_part_off_{i}"]) for i in range(3)]
    assert offs[0] == 0 and all(o % 4096 == 0 for o in offs) and offs == [0, parts[0].size, parts[0].size + parts[1].size]

    # metadata only, for the array a build left behind
    sa40.tofile(os.path.join(tmp, "native.sa40"))
    idxm = os.path.join(tmp, "idxm")
    r = subprocess.run([tool, "--meta-only", "--sa", os.path.join(tmp, "native.sa40"), "--index-dir", idxm] + common, capture_output=True, text=True)
    assert r.returncode == 0 and "order spot-check passed" in r.stderr
    assert _kv(open(os.path.join(idxm, "index.meta")).read())["sa_part_0"] == os.path.join(tmp, "native.sa40")

    # widening returns the 64-bit entries
    r = subprocess.run([tool, "--widen", "--in", os.path.join(tmp, "native.sa40"), "--out", os.path.join(tmp, "back.u64")], capture_output=True, text=True)
    assert r.returncode == 0 and np.array_equal(np.fromfile(os.path.join(tmp, "back.u64"), dtype="<u8"), sa64)

    # refusals: a duplicate entry, an entry out of range, two entries out of order, a bad command line
    bad = sa64.copy(); bad[7] = bad[8]
    bad.tofile(os.path.join(tmp, "dup.u64"))
    r = subprocess.run([tool, "--in", os.path.join(tmp, "dup.u64"), "--index-dir", os.path.join(tmp, "x1")] + common, capture_output=True, text=True)
    assert r.returncode == 1 and "not a permutation" in r.stderr
    bad = sa64.copy(); bad[5] = n
    bad.tofile(os.path.join(tmp, "range.u64"))
    r = subprocess.run([tool, "--in", os.path.join(tmp, "range.u64"), "--index-dir", os.path.join(tmp, "x2"), "--check", "range"] + common, capture_output=True, text=True)
    assert r.returncode == 1 and "out of range" in r.stderr
    bad = sa64.copy(); bad[[100, 101]] = bad[[101, 100]]
    bad.tofile(os.path.join(tmp, "swap.u64"))
    r = subprocess.run([tool, "--in", os.path.join(tmp, "swap.u64"), "--index-dir", os.path.join(tmp, "x3"), "--spot", str(n)] + common, capture_output=True, text=True)
    assert r.returncode == 1 and "order violated" in r.stderr and not os.path.exists(os.path.join(tmp, "x3", "index.meta"))
    r = subprocess.run([tool, "--meta-only", "--text", os.path.join(tmp, "text.u16"), "--sym-bytes", "2", "--index-dir", tmp], capture_output=True, text=True)
    assert r.returncode == 2 and "--sa" in r.stderr and "usage" in r.stderr


@pytest.mark.gpu
def test_cascade_and_query_find_against_the_oracle(tmp_path, oracle):
    from cascade_b200 import api
    tmp = str(tmp_path)
    n = 300000
    T = api.gen_corpus_host(n, 2, 256)[:n]
    _write_index(tmp, T)
    env = dict(os.environ, GPU_SACA_P_TARGET="8", CASCADE_VALIDATE="1")
    r = subprocess.run([os.path.join(BIN, "cascade"), os.path.join(tmp, "text.u16"), os.path.join(tmp, "text.sa40")], capture_output=True, text=True, env=env)
    assert r.returncode == 0, r.stderr
    got = np.fromfile(os.path.join(tmp, "text.sa40"), dtype=np.uint8)
    want = oracle.build_sa40(T)
    assert got.size == 5 * n and np.array_equal(got, want[:5 * n])

    # the same file from a build sharded over in-process ranks (threads share the GPU when the box has only one)
    for gpus in ("2", "3"):
        out2 = os.path.join(tmp, f"text.g{gpus}.sa40")
        r = subprocess.run([os.path.join(BIN, "cascade"), os.path.join(tmp, "text.u16"), out2], capture_output=True, text=True,
                           env=dict(env, CASCADE_GPUS=gpus))
        assert r.returncode == 0, r.stderr
        assert np.array_equal(np.fromfile(out2, dtype=np.uint8), want[:5 * n]), gpus

    # the reference's knobs: the lower tier forced (the build then runs part by part with its lists in host memory, parts capped
    # as the reference's test knob caps its slabs); a host budget that the build would pass refuses it before it starts, unless
    # there are scratch directories, over which the lists of the parts beyond the budget are then striped as files
    out3 = os.path.join(tmp, "text.parts.sa40")
    r = subprocess.run([os.path.join(BIN, "cascade"), os.path.join(tmp, "text.u16"), out3], capture_output=True, text=True,
                       env=dict(env, GPU_SACA_FORCE_SPILL="1", GPU_SACA_CHUNK_CAP="70000"))
    assert r.returncode == 0 and "part by part" in r.stderr and "of 0 parts in files" in r.stderr, r.stderr
    assert np.array_equal(np.fromfile(out3, dtype=np.uint8), want[:5 * n])
    os.remove(out3)
    r = subprocess.run([os.path.join(BIN, "cascade"), os.path.join(tmp, "text.u16"), out3], capture_output=True, text=True,
                       env=dict(env, GPU_SACA_FORCE_SPILL="1", GPU_SACA_RAM_BUDGET="100000"))
    assert r.returncode != 0 and "GPU_SACA_RAM_BUDGET" in r.stderr and "GPU_SACA_SCRATCH" in r.stderr
    roots = [os.path.join(tmp, "scratch_a"), os.path.join(tmp, "scratch_b")]
    for d in roots:
        os.mkdir(d)
    r = subprocess.run([os.path.join(BIN, "cascade"), os.path.join(tmp, "text.u16"), out3], capture_output=True, text=True,
                       env=dict(env, GPU_SACA_FORCE_SPILL="1", GPU_SACA_CHUNK_CAP="70000", GPU_SACA_RAM_BUDGET="500000", GPU_SACA_SCRATCH=":".join(roots)))
    assert r.returncode == 0 and "parts in files" in r.stderr and "of 0 parts in files" not in r.stderr, r.stderr
    assert np.array_equal(np.fromfile(out3, dtype=np.uint8), want[:5 * n])
    assert all(os.listdir(d) == [] for d in roots)

    q = os.path.join(tmp, "a.qry")
    assert subprocess.run([os.path.join(BIN, "query"), "gen", "--index", tmp, "--out", q, "--kind", "substring", "--q", "5000", "--len", "1,2,4,8,16",
                           "--seed", "1"], capture_output=True).returncode == 0
    r = subprocess.run([os.path.join(BIN, "query"), "find", "--index", tmp, "--queries", q, "--reps", "2", "--validate", "--locate", "100",
                        "--itv-out", os.path.join(tmp, "a.itv"), "--cnt-dir", tmp, "--pos-out", os.path.join(tmp, "a.pos")], capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    kv = _kv(r.stdout)
    off, sym, _ = _read_qry(q)
    want_itv = oracle.find_batch(T, want, off, sym)
    itv = np.fromfile(os.path.join(tmp, "a.itv"), dtype="<u8")
    cnt = np.fromfile(os.path.join(tmp, "a.cnt"), dtype="<u8")
    assert np.array_equal(itv, want_itv) and np.array_equal(cnt, want_itv[1::2] - want_itv[0::2])
    assert kv["validate"] == "ok" and int(kv["counts_hash"], 16) == oracle.counts_hash(want_itv)
    # the same array split into two parts by sa_convert answers the same
    tool = os.path.join(BIN, "sa_convert")
    assert subprocess.run([tool, "--widen", "--in", os.path.join(tmp, "text.sa40"), "--out", os.path.join(tmp, "text.u64")], capture_output=True).returncode == 0
    idx2 = os.path.join(tmp, "idx2")
    r2 = subprocess.run([tool, "--in", os.path.join(tmp, "text.u64"), "--text", os.path.join(tmp, "text.u16"), "--sym-bytes", "2", "--index-dir", idx2, "--parts", "2",
                         "--part-dirs", os.path.join(tmp, "p0") + ":" + os.path.join(tmp, "p1"), "--sep", "65535"], capture_output=True, text=True)
    assert r2.returncode == 0, r2.stderr
    r2 = subprocess.run([os.path.join(BIN, "query"), "find", "--index", idx2, "--queries", q, "--reps", "1"], capture_output=True, text=True)
    assert r2.returncode == 0, r2.stderr
    assert _kv(r2.stdout)["counts_hash"] == kv["counts_hash"]
    blob = np.fromfile(os.path.join(tmp, "a.pos"), dtype="<u8")
    qn, total = int(blob[0]), int(blob[1])
    poff, pos = blob[2:2 + qn + 1], blob[2 + qn + 1:]
    wp, wc = oracle.locate_batch(want, want_itv, 100)
    assert qn == 5000 and total == int(wc.sum()) == pos.size
    for i in range(0, qn, 53):
        assert np.array_equal(pos[int(poff[i]):int(poff[i + 1])], wp[i, :wc[i]])
