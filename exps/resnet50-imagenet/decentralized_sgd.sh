#!/bin/bash
# ResNet-50 on ImageNet with D-PSGD on a ring (dl_code/exps/finetune-resnet50-imagenet/decentralized_sgd.sh:1-14).
PY=${PYTHON:-python}
$PY -m chocosgd_b200.run --arch resnet50 --optimizer sgd --experiment test \
    --data imagenet --use_lmdb_data True --data_dir ./data/ILSVRC --pin_memory True --dtype bf16 \
    --batch_size 128 --base_batch_size 256 --num_workers 8 \
    --num_epochs 90 --partition_data random --reshuffle_per_epoch True --stop_criteria epoch \
    --on_cuda True --n_mpi_process 8 --n_sub_process 1 --world 0,1,2,3,4,5,6,7 \
    --lr 0.1 --lr_scaleup True --lr_scaleup_factor graph --lr_warmup True --lr_warmup_epochs 5 \
    --lr_schedule_scheme custom_multistep --lr_change_epochs 30,60,80 \
    --weight_decay 1e-4 --use_nesterov True --momentum_factor 0.9 \
    --graph_topology ring --hostfile hostfile --backend nccl --summary_freq 100
