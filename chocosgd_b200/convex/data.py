"""Data for the convex experiments: the synthetic benchmark problem, LIBSVM -> dense pickle
conversion (``convex_code/pickle_datasets.py:8-24``) and pickle helpers (``convex_code/utils.py``)."""
from __future__ import annotations

import os
import pickle

import numpy as np


def synthetic_logistic(num_samples=40000, num_features=2000, seed=0, noise=0.1):
    """Rows ~ N(0, I) normalised to unit L2 norm; labels sign(x.w* + noise eps), w* ~ N(0, I)."""
    rs = np.random.RandomState(seed)
    A = rs.randn(num_samples, num_features)
    A /= np.linalg.norm(A, axis=1, keepdims=True)
    w = rs.randn(num_features)
    y = np.sign(A @ w + noise * rs.randn(num_samples))
    y[y == 0] = 1.0
    return A, y


def pickle_libsvm(in_path, out_path, n_features=None):
    """Dense (A, y) pickle of a LIBSVM file (epsilon, rcv1)."""
    from sklearn.datasets import load_svmlight_file

    A, y = load_svmlight_file(in_path, n_features=n_features)
    with open(out_path, "wb") as f:
        pickle.dump((A.toarray() if hasattr(A, "toarray") else A, y), f, protocol=pickle.HIGHEST_PROTOCOL)


def pickle_it(var, name, directory):
    os.makedirs(directory, exist_ok=True)
    with open(os.path.join(directory, "{}.pickle".format(name)), "wb") as f:
        pickle.dump(var, f)


def unpickle_dir(d):
    out = {}
    for fn in os.listdir(d):
        if fn.endswith(".pickle"):
            with open(os.path.join(d, fn), "rb") as f:
                out[fn[:-7]] = pickle.load(f)
    return out


def main(argv=None):
    """``python -m chocosgd_b200.convex.data <libsvm file> <out.pickle>`` or
    ``python -m chocosgd_b200.convex.data --synthetic <out.pickle> [N d]``."""
    import sys

    argv = list(sys.argv[1:] if argv is None else argv)
    if argv and argv[0] == "--synthetic":
        n, d = (int(argv[2]), int(argv[3])) if len(argv) >= 4 else (40000, 2000)
        with open(argv[1], "wb") as f:
            pickle.dump(synthetic_logistic(n, d), f, protocol=pickle.HIGHEST_PROTOCOL)
    elif len(argv) == 2:
        pickle_libsvm(argv[0], argv[1])
    else:
        raise SystemExit(main.__doc__)


if __name__ == "__main__":
    main()
