#!/bin/bash
# LSTM language model on WikiText-2 (the reference's dl_code/exps/finetune-lstm/example.sh:1-13):
# 3 x 650 LSTM, tied weights, bptt 30, clip 0.4, dropout 0.4, batch 32 per rank.
# `--data synthetic_wikitext2` draws uniform token ids of the same vocabulary size (33 278).
PY=${PYTHON:-python}
COMMON="--arch rnn_lm --rnn_n_hidden 650 --rnn_n_layers 3 --rnn_bptt_len 30 --rnn_clip 0.4 \
    --rnn_use_pretrained_emb False --rnn_tie_weights True --drop_rate 0.40 --experiment test \
    --data wikitext2 --data_dir ./data --batch_size 32 --base_batch_size 24 --num_workers 2 \
    --num_epochs 300 --partition_data random --reshuffle_per_epoch False --stop_criteria epoch \
    --n_mpi_process 8 --n_sub_process 1 --world 0,1,2,3,4,5,6,7 --on_cuda True \
    --lr 2.5 --lr_scaleup True --lr_scaleup_factor graph --lr_warmup True --lr_warmup_epochs 5 \
    --lr_schedule_scheme custom_multistep --lr_change_epochs 150,225 --lr_decay 10 \
    --weight_decay 0 --use_nesterov False --momentum_factor 0 --hostfile hostfile --backend nccl"

# decentralized SGD, ring
$PY -m chocosgd_b200.run $COMMON --optimizer sgd --graph_topology ring

# CHOCO-SGD with QSGD (16 levels), ring
$PY -m chocosgd_b200.run $COMMON --optimizer parallel_choco_v --graph_topology ring \
    --comm_op quantize_qsgd --quantize_level 4 --is_biased True --consensus_stepsize 0.3
