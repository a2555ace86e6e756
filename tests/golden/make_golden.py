"""Writes the golden vectors under tests/golden/ by running the reference's own CPU code (oracle/_ref/libcascade_ref.so,
compiled from the reference's sources by oracle/Makefile). Run in a container that has the reference tree:

    make -C oracle REF=<reference tree> && python tests/golden/make_golden.py

Outputs:
  known_answers.json   the reference's known-answer table of (text, pattern, count) (its test_edge_cases), each with the
                       interval that the reference's ref::find_one returns over the reference's build_sa40 array
  sa_fixtures.npz      for every small fixture text: the text and the suffix array from the reference's build_sa40
  query_fixtures.npz   for some fixture texts: a query batch and the intervals from the reference's host_search::find
"""
import json
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
import conftest  # noqa: E402

# (text, pattern, count): the cases of the reference's known-answer test, read from its test source as data.
KNOWN = [
    ([0, 0, 0, 0], [], 4), ([0, 0, 0, 0], [0], 4), ([0, 0, 0, 0], [0, 0, 0, 0], 1), ([0, 0, 0, 0], [0, 0, 0, 0, 0], 0),
    ([5, 3, 5, 0], [0], 1), ([5, 3, 5, 0], [0, 0], 0), ([5, 3, 5, 0], [5, 0], 1), ([5, 3, 5, 0], [5, 0, 0], 0),
    ([9, 8, 7], [7, 0], 0), ([3, 4, 5], [1], 0), ([3, 4, 5], [3, 1], 0), ([3, 4, 5], [9], 0), ([3, 4, 5], [5, 5], 0),
    ([65535, 1, 65535, 1, 65535], [65535], 3), ([65535, 1, 65535, 1, 65535], [1, 65535], 2), ([65535, 65535], [65535, 65535, 65535], 0),
]


def main():
    ref = conftest.Oracle(conftest.REF_LIB, "ref_")
    known = []
    for T, P, count in KNOWN:
        Ta, Pa = np.array(T, np.uint16), np.array(P, np.uint16)
        sa = ref.build_sa40(Ta)
        lo, hi = ref.find_one(Ta, sa, Pa)
        assert hi - lo == count, (T, P, count, lo, hi)
        assert ref.brute_find(Ta, Pa) == (lo, hi)
        known.append({"text": T, "pattern": P, "count": count, "lo": lo, "hi": hi, "sa": [int(x) for x in conftest.sa40_to_u64(sa, len(T))]})
    with open(os.path.join(HERE, "known_answers.json"), "w") as f:
        json.dump(known, f, indent=0)

    texts = conftest.fixture_texts()
    sa_out = {}
    for name, T in texts.items():
        sa = ref.build_sa40(T)
        assert ref.is_correct(T, sa)
        sa_out["T_" + name] = T
        sa_out["SA_" + name] = conftest.sa40_to_u64(sa, len(T)).astype(np.uint32)
    np.savez_compressed(os.path.join(HERE, "sa_fixtures.npz"), **sa_out)

    q_out = {}
    rng = np.random.default_rng(11)
    for name in ("rand_n1000_s2", "rand_n1000_s4", "rand_n20000_s16", "rand_n20000_s65536", "periodic_ab", "fibonacci", "all_zero_1000",
                 "binary_zero_tail", "corner_case", "rand_n17_s3"):
        T = texts[name]
        sa = ref.build_sa40(T)
        off, sym, _ = conftest.fixture_queries(T, rng, 200)
        itv = ref.find_batch(T, sa, off, sym, threads=2)
        q_out["off_" + name] = off
        q_out["sym_" + name] = sym
        q_out["itv_" + name] = itv
    np.savez_compressed(os.path.join(HERE, "query_fixtures.npz"), **q_out)
    print("golden vectors written")


if __name__ == "__main__":
    main()
