"""Flat packing of a list of tensors (``dl_code/pcode/utils/tensor_buffer.py:5-40``).

Kept for API parity and for code outside the hot path; the optimizers themselves never
pack per step because the model parameters already *are* views of one flat arena
(see ``optim/arena.py``)."""
import torch


class TensorBuffer:
    def __init__(self, tensors, use_cuda=None):
        tensors = list(tensors)
        sizes = [t.nelement() for t in tensors]
        self._start_idx = [0] * len(tensors)
        self._end_idx = [0] * len(tensors)
        end = 0
        for i, n in enumerate(sizes):
            self._start_idx[i] = end
            end += n
            self._end_idx[i] = end
        self._tensors_len = len(tensors)
        self._tensors_sizes = [t.size() for t in tensors]
        self.buffer = torch.cat([t.reshape(-1) for t in tensors]) if tensors else torch.empty(0)

    def __getitem__(self, index):
        return self.buffer[self._start_idx[index]:self._end_idx[index]].view(self._tensors_sizes[index])

    def __len__(self):
        return self._tensors_len

    def is_cuda(self):
        return self.buffer.is_cuda

    def nelement(self):
        return self.buffer.nelement()

    def unpack(self, tensors):
        for tensor, entry in zip(tensors, self):
            tensor.data[:] = entry
