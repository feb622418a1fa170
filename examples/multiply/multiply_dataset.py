"""python examples/multiply/multiply_dataset.py --out ~/data/multiply [--digits 2] [--n 4096]"""

import argparse
import os
import random

import pandas as pd


def rows(n: int, digits: int, seed: int):
    rng = random.Random(seed)
    lo, hi = 10 ** (digits - 1), 10 ** digits - 1
    for i in range(n):
        a, b = rng.randint(lo, hi), rng.randint(lo, hi)
        yield {"prompt": [{"role": "user", "content": f"What is {a} times {b}? Answer with the number only."}],
               "env_class": "multiply", "reward_spec": {"method": "rule", "ground_truth": str(a * b)}, "uid": f"m{seed}-{i}"}


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--out", default=os.path.expanduser("~/data/multiply"))
    ap.add_argument("--digits", type=int, default=2)
    ap.add_argument("--n", type=int, default=4096)
    a = ap.parse_args()
    os.makedirs(a.out, exist_ok=True)
    pd.DataFrame(list(rows(a.n, a.digits, 0))).to_parquet(os.path.join(a.out, "train.parquet"))
    pd.DataFrame(list(rows(max(16, a.n // 16), a.digits, 1))).to_parquet(os.path.join(a.out, "validation.parquet"))
