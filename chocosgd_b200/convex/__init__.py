"""Decentralized logistic-regression simulator (the convex experiments of the CHOCO paper):
``n_cores`` simulated nodes in one process running plain gossip / CHOCO / DCD-PSGD / ECD-PSGD
with top-k, random-k or QSGD compression (``convex_code/`` of the reference)."""
from .logistic import LogisticDecentralizedSGD, mixing_matrix_convex, qsgd_quantize
from .parameters import Parameters
