"""Dictionary with element-wise arithmetic over its values
(``dl_code/pcode/utils/mathdict.py``; unused by the training path, kept for parity)."""
from numbers import Number


class MathDict:
    def __init__(self, dictionary):
        self.dictionary = dict(dictionary)
        self.keys = set(self.dictionary.keys())

    def __str__(self):
        return f"MathDict({self.dictionary})"

    __repr__ = __str__

    def __getitem__(self, key):
        return self.dictionary[key]

    def map(self, mapfun):
        return MathDict({k: mapfun(k, v) for k, v in self.dictionary.items()})

    def filter(self, condfun):
        return MathDict({k: v for k, v in self.dictionary.items() if condfun(k, v)})

    def detach(self):
        for v in self.dictionary.values():
            v.detach_()

    def values(self):
        return self.dictionary.values()

    def items(self):
        return self.dictionary.items()

    def _binary(self, other, fn):
        if isinstance(other, MathDict):
            assert other.keys == self.keys
            return MathDict({k: fn(self.dictionary[k], other.dictionary[k]) for k in self.keys})
        if isinstance(other, Number):
            return MathDict({k: fn(self.dictionary[k], other) for k in self.keys})
        return NotImplemented

    def __add__(self, other):
        return self._binary(other, lambda a, b: a + b)

    __radd__ = __add__

    def __sub__(self, other):
        return self._binary(other, lambda a, b: a - b)

    def __mul__(self, other):
        return self._binary(other, lambda a, b: a * b)

    __rmul__ = __mul__

    def __truediv__(self, other):
        return self._binary(other, lambda a, b: a / b)

    def __neg__(self):
        return MathDict({k: -v for k, v in self.dictionary.items()})
