#!/bin/bash
# The epsilon sweep of the convex code (convex_code/experiment_epsilon_final.py:24-315): 9 nodes on a
# ring, 10 epochs, 5 seeds, random and label-sorted splits, exact / CHOCO / DCD / ECD with their compressors.
# 1. python -m chocosgd_b200.convex.data  <epsilon_normalized LIBSVM file> data/epsilon.pickle
# 2. python -m chocosgd_b200.convex.baselines data/epsilon.pickle dump/optimum-epsilon
PY=${PYTHON:-python}
$PY -m chocosgd_b200.convex.experiment final --dataset data/epsilon.pickle --out dump/epsilon-final --nproc 10
$PY -m chocosgd_b200.tools.plot_convex dump/epsilon-final --baseline dump/optimum-epsilon/baselines.pickle --out plots
