#!/bin/bash
# ResNet-20 on CIFAR-10, 8 ranks on one 8 x B200 node (one rank per GPU), 300 epochs.
# Same recipes as the reference's dl_code/exps/finetune-resnet20-cifar10/example.sh:1-87: the
# flags carry over unchanged; `--data synthetic_cifar10` runs the same shapes without a dataset.
PY=${PYTHON:-python}
COMMON="--arch resnet20 --experiment test --data cifar10 --data_dir ./data --pin_memory True \
    --batch_size 128 --num_workers 2 --num_epochs 300 --partition_data random --reshuffle_per_epoch True \
    --stop_criteria epoch --n_mpi_process 8 --n_sub_process 1 --world 0,1,2,3,4,5,6,7 --on_cuda True \
    --lr 0.1 --lr_scaleup True --lr_scaleup_factor graph --lr_warmup True --lr_warmup_epochs 5 \
    --lr_schedule_scheme custom_multistep --lr_change_epochs 150,225 \
    --weight_decay 1e-4 --use_nesterov True --momentum_factor 0.9 \
    --hostfile hostfile --backend nccl --evaluate_consensus True"

# centralized SGD, complete topology (gradient all-reduce + update in one kernel)
$PY -m chocosgd_b200.run $COMMON --optimizer sgd --base_batch_size 64 --graph_topology complete

# decentralized SGD (D-PSGD), ring topology
$PY -m chocosgd_b200.run $COMMON --optimizer sgd --base_batch_size 64 --graph_topology ring

# CHOCO-SGD with sign + norm compression, ring topology
$PY -m chocosgd_b200.run $COMMON --optimizer parallel_choco --base_batch_size 24 --graph_topology ring \
    --comm_op sign --consensus_stepsize 0.45

# CHOCO-SGD with top-1 % sparsification, ring topology
$PY -m chocosgd_b200.run $COMMON --optimizer parallel_choco_v --base_batch_size 24 --graph_topology ring \
    --comm_op compress_top_k --compress_ratio 0.99 --consensus_stepsize 0.02

# DCD-PSGD with 4-bit QSGD, ring topology
$PY -m chocosgd_b200.run $COMMON --optimizer dcd_psgd --base_batch_size 64 --graph_topology ring \
    --comm_op quantize_qsgd --quantize_level 4 --is_biased False

# ECD-PSGD with 4-bit QSGD, ring topology
$PY -m chocosgd_b200.run $COMMON --optimizer ecd_psgd --base_batch_size 64 --graph_topology ring \
    --comm_op quantize_qsgd --quantize_level 4 --is_biased False

# DeepSqueeze with sign + norm, ring topology
$PY -m chocosgd_b200.run $COMMON --optimizer deep_squeeze --base_batch_size 64 --graph_topology ring \
    --comm_op sign --consensus_stepsize 0.04

# Deep Gradient Compression (centralized), top-0.1 % with the sparsity warm-up
$PY -m chocosgd_b200.run $COMMON --optimizer dgc --base_batch_size 64 --graph_topology complete \
    --comm_op compress_top_k --compress_ratio 0.999 --compress_warmup_epochs 4 --mask_momentum True

# EF-signSGD (centralized)
$PY -m chocosgd_b200.run $COMMON --optimizer ef_sign_sgd --base_batch_size 64 --graph_topology complete \
    --comm_op sign
