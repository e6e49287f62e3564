"""Hand-written sm_100a kernels (``csrc/``) and their Python bindings.

``_lib``      ctypes loader of the in-tree shared library
``sgd``       fused multi-segment Nesterov / momentum / weight-decay update
``compress``  stand-alone sign pack/unpack, top-k, random-k, QSGD kernels
``gossip``    fused CHOCO step kernels with in-kernel NVLink push (the product path)
``gemm``      tcgen05 / TMEM GEMM
``nn``        layer classes used by the model zoo (conv / batch-norm / linear / LSTM)
"""
