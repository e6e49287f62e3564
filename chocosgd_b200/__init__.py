"""B200-native decentralized training with compressed gossip (CHOCO-SGD family).

Sub-packages
------------
config      command line surface (same flag names as the reference's ``dl_code/parameters.py``)
parallel    mixing topologies, process-group bootstrap, peer-mapped symmetric arenas, aggregators
compress    top-k / random-k / QSGD / sign operators (CPU oracles + wire formats)
ops         ctypes bindings of the hand-written sm_100a kernels and their autograd wrappers
optim       the eight distributed algorithms (CHOCO, D-PSGD, DCD, ECD, DeepSqueeze, DGC, EF-sign, SGD)
models      ResNet (cifar/imagenet), RNN LM, DenseNet, WideResNet, VGG, LeNet, MLP
data        synthetic + on-disk datasets, seeded partitioner
train       CV / NLP loops, LR scheduler, metrics
utils       timer, JSON logger, trackers, checkpoints, error handling
tools       result extraction, plotting, consensus step-size tuner
convex      decentralized logistic-regression simulator (numpy oracle + CUDA path)
sim         matrix-form multi-node simulator of every algorithm (the test oracle)
"""

__version__ = "0.1.0"
