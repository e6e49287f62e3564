"""Optimal regularised logistic loss f* with scikit-learn (``convex_code/baselines.py:12-36``):
``SGDClassifier(loss="log_loss", alpha=lambda, tol=1e-5)``; the training sub-optimality curves
are plotted against this value."""
from __future__ import annotations

import numpy as np


def regularised_loss(clf, A, y, reg):
    w = clf.coef_.ravel()
    z = -y * (A @ w + clf.intercept_[0])
    return float(np.logaddexp(0.0, z).mean() + reg * np.square(w).sum() / 2)


def optimum(A, y, reg=None, seed=0, max_iter=2000):
    from sklearn.linear_model import SGDClassifier

    reg = 1.0 / A.shape[0] if reg is None else reg
    clf = SGDClassifier(loss="log_loss", penalty="l2", alpha=reg, tol=1e-5, max_iter=max_iter, fit_intercept=False,
                        random_state=seed, n_iter_no_change=20)
    clf.fit(A, y)
    return regularised_loss(clf, A, y, reg), clf


def main(argv=None):
    """``python -m chocosgd_b200.convex.baselines <data.pickle> <out dir>`` writes ``baselines.pickle``
    (the optimal loss f*, as ``convex_code/baselines.py:24-36`` does for epsilon)."""
    import pickle
    import sys

    from .data import pickle_it

    argv = list(sys.argv[1:] if argv is None else argv)
    if len(argv) != 2:
        raise SystemExit(main.__doc__)
    with open(argv[0], "rb") as f:
        A, y = pickle.load(f)
    best, _ = optimum(A, y)
    pickle_it(best, "baselines", argv[1])
    print("optimal regularised loss:", best)


if __name__ == "__main__":
    main()
