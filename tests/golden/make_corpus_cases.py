"""Generates tests/golden/reference_corpus_cases.json: the test descriptions that the reference's own config files
expand to, for the GPU test that has no checkout of the reference to read (tests/test_gpu_reference_corpus.py).

Run where the reference checkout is present:

    python tests/golden/make_corpus_cases.py

Each listed file of mme/mme_verification/*/configs is read with this repository's parser of the reference's test-config
format (intel_gaudi3_software_b200/config_runner.py; seeded, so "random" values are fixed here), and every expanded test
is stored as the keys in which it differs from the format's defaults. Tests on data types outside the backend (fp16)
are listed by name under "rejected". Nothing but shapes, types, flags and value ranges is taken from the files.
"""
import json
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

from intel_gaudi3_software_b200 import config_runner as cr  # noqa: E402
from oracle.oracle import reference_root  # noqa: E402

SEED = 7
FILES = ["gaudi3/configs/basic_tests/basic_%s.json" % n for n in
         ("fwd", "dedx", "dedw", "ab", "abt", "atb", "atbt", "ab_strides", "fwd_strides", "dual_gemm")] + [
    "gaudi3/configs/numerics/numerics_fp8.json", "gaudi2/configs/stochastic_rounding.json"]
# chip model the reference's test manager would run each directory's files on
CHIP = {"gaudi3": 2, "gaudi2": 1}


def main():
    root = reference_root()
    if root is None:
        sys.exit("no checkout of the reference here")
    base = os.path.join(root, "mme", "mme_verification")
    default = cr.default_test()
    out = {"seed": SEED, "files": {}}
    for rel in FILES:
        doc = cr.load_config(os.path.join(base, rel))
        tests, rejected = [], []
        for test in doc["tests"]:
            try:
                parsed = cr.Parser(SEED + len(tests)).parse({"tests": [test]})
            except cr.ConfigError as e:
                name = next((list(i.values())[0][0] for i in test if "testName" in i), "?")
                rejected.append({"name": name, "why": str(e)})
                continue
            for t in parsed:
                t.pop("ignored", None)
                tests.append({k: v for k, v in t.items() if default.get(k, object()) != v})
        out["files"][rel] = {"chip": CHIP[rel.split("/")[0]], "tests": tests, "rejected": rejected}
        print("%-55s %4d tests, %d rejected" % (rel, len(tests), len(rejected)))
    path = os.path.join(ROOT, "tests", "golden", "reference_corpus_cases.json")
    with open(path, "w") as f:
        json.dump(out, f, separators=(",", ":"), sort_keys=True)
    print("wrote", path, os.path.getsize(path), "bytes")


if __name__ == "__main__":
    main()
