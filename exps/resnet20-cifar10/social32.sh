#!/bin/bash
# CHOCO-SGD with sign + norm on the 32-node social graph (4 ranks per GPU of one 8-GPU node):
# the reference's recipe of dl_code/exps/finetune-resnet20-cifar10/example.sh:44-57.  More than one
# rank per GPU uses the torch.distributed transport (`--gossip_impl nccl` is not possible with
# several ranks on a device, so the backend is gloo and the gossip runs through send / recv).
PY=${PYTHON:-python}
$PY -m chocosgd_b200.run --arch resnet20 --optimizer parallel_choco --experiment test \
    --data cifar10 --data_dir ./data --batch_size 128 --base_batch_size 64 --num_workers 0 \
    --num_epochs 300 --partition_data random --reshuffle_per_epoch True --stop_criteria epoch \
    --n_mpi_process 32 --n_sub_process 1 \
    --world 0,0,0,0,1,1,1,1,2,2,2,2,3,3,3,3,4,4,4,4,5,5,5,5,6,6,6,6,7,7,7,7 --on_cuda True \
    --lr 0.1 --lr_scaleup True --lr_scaleup_factor graph --lr_warmup True --lr_warmup_epochs 5 \
    --lr_schedule_scheme custom_multistep --lr_change_epochs 150,225 \
    --weight_decay 1e-4 --use_nesterov True --momentum_factor 0.9 \
    --comm_op sign --consensus_stepsize 0.5 --graph_topology social --backend gloo --gossip_impl nccl
