"""Datasets, partitioning and loaders (``dl_code/pcode/create_dataset.py``,
``dl_code/pcode/datasets/``)."""
from .loaders import define_dataset, load_data_batch
from .partition import DataPartitioner, Partition
from .synthetic import SyntheticImages, SyntheticTokens
