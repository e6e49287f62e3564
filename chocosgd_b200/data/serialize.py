"""Packing datasets into one random-access file, and reading them back.

The reference serialises ImageNet (encoded JPEG bytes + label) and the epsilon / rcv1 feature
sets into LMDB files keyed by index, with the key list under ``__keys__`` and the count under
``__len__`` (``dl_code/pcode/datasets/loader/serialize.py:1-88``,
``dl_code/pcode/datasets/loader/utils.py:30-204``).  ``write_records`` produces the same layout
when the ``lmdb`` package is available (path ending in ``.lmdb``); any other path gets a
dependency-free record file (``RecordFile``: one data blob + an offset table) with the same
key / value contract, so the tooling also works where ``lmdb`` cannot be installed.

    python -m chocosgd_b200.data.serialize --folder <ImageFolder root> --split train --out train.lmdb
    python -m chocosgd_b200.data.serialize --libsvm epsilon_normalized --out epsilon_train.lmdb
"""
from __future__ import annotations

import argparse
import os
import pickle
import struct
from typing import Iterable, Tuple

import numpy as np

MAGIC = b"CHOCOREC1"


def dumps(obj) -> bytes:
    """msgpack when installed (the reference's format, numpy arrays as raw bytes), pickle otherwise."""
    try:
        import msgpack

        def enc(o):
            if isinstance(o, np.ndarray):
                return {"__nd__": True, "dtype": str(o.dtype), "shape": list(o.shape), "data": o.tobytes()}
            raise TypeError(type(o))

        return b"M" + msgpack.packb(obj, default=enc, use_bin_type=True)
    except ImportError:
        return b"P" + pickle.dumps(obj, protocol=4)


def loads(buf: bytes):
    tag, body = buf[:1], buf[1:]
    if tag == b"M":
        import msgpack

        def dec(o):
            if o.get("__nd__"):
                return np.frombuffer(o["data"], dtype=o["dtype"]).reshape(o["shape"])
            return o

        return msgpack.unpackb(body, object_hook=dec, raw=False)
    if tag == b"P":
        return pickle.loads(body)
    try:  # files written by the reference's tool: untagged msgpack / pyarrow
        import msgpack

        return msgpack.loads(buf, raw=False)
    except Exception:
        return pickle.loads(buf)


class RecordFile:
    """``MAGIC | n | offsets[n + 1] | blobs``: values addressed by integer index, read with ``pread``."""

    def __init__(self, path):
        self.path = path
        self.fd = os.open(path, os.O_RDONLY)
        head = os.pread(self.fd, len(MAGIC) + 8, 0)
        if head[:len(MAGIC)] != MAGIC:
            raise ValueError(f"{path} is not a record file")
        (self.n,) = struct.unpack("<q", head[len(MAGIC):])
        table = os.pread(self.fd, 8 * (self.n + 1), len(MAGIC) + 8)
        self.offsets = np.frombuffer(table, dtype="<i8")
        self.base = len(MAGIC) + 8 + 8 * (self.n + 1)

    def __len__(self):
        return self.n

    def get(self, i: int) -> bytes:
        a, b = int(self.offsets[i]), int(self.offsets[i + 1])
        return os.pread(self.fd, b - a, self.base + a)

    def close(self):
        if self.fd is not None:
            os.close(self.fd)
            self.fd = None

    @staticmethod
    def write(path, blobs: Iterable[bytes]):
        tmp = path + ".data"
        offsets = [0]
        with open(tmp, "wb") as f:
            for b in blobs:
                f.write(b)
                offsets.append(offsets[-1] + len(b))
        n = len(offsets) - 1
        with open(path, "wb") as out, open(tmp, "rb") as f:
            out.write(MAGIC + struct.pack("<q", n) + np.asarray(offsets, dtype="<i8").tobytes())
            while True:
                chunk = f.read(1 << 24)
                if not chunk:
                    break
                out.write(chunk)
        os.remove(tmp)
        return n


class RecordStore:
    """Read access by index to either layout."""

    def __init__(self, path):
        self.path = path
        self._lmdb = self._file = None
        if path.endswith(".lmdb") and not _is_record_file(path):
            import lmdb

            self._lmdb = lmdb.open(path, subdir=os.path.isdir(path), readonly=True, lock=False, readahead=False,
                                   meminit=False)
            with self._lmdb.begin(write=False) as txn:
                self.length = loads(txn.get(b"__len__"))
                self.keys = loads(txn.get(b"__keys__"))
        else:
            self._file = RecordFile(path)
            self.length = len(self._file)

    def __len__(self):
        return self.length

    def __getitem__(self, i):
        if self._file is not None:
            return loads(self._file.get(i))
        with self._lmdb.begin(write=False) as txn:
            return loads(txn.get(self.keys[i]))


def _is_record_file(path):
    try:
        with open(path, "rb") as f:
            return f.read(len(MAGIC)) == MAGIC
    except (IsADirectoryError, FileNotFoundError):
        return False


def write_records(path, records: Iterable[Tuple[object, int]], write_frequency=5000, map_size=1 << 40, use_lmdb=None):
    """``records`` yields ``(payload, label)``; returns the number written."""
    if use_lmdb is None:
        use_lmdb = path.endswith(".lmdb")
        if use_lmdb:
            try:
                import lmdb  # noqa: F401
            except ImportError:
                use_lmdb = False
    if not use_lmdb:
        return RecordFile.write(path, (dumps((payload, int(label))) for payload, label in records))
    import lmdb

    db = lmdb.open(path, subdir=False, map_size=map_size, readonly=False, meminit=False, map_async=True)
    txn, n = db.begin(write=True), 0
    for payload, label in records:
        txn.put("{}".format(n).encode("ascii"), dumps((payload, int(label))))
        n += 1
        if n % write_frequency == 0:
            txn.commit()
            txn = db.begin(write=True)
    txn.commit()
    with db.begin(write=True) as txn:
        txn.put(b"__keys__", dumps(["{}".format(k).encode("ascii") for k in range(n)]))
        txn.put(b"__len__", dumps(n))
    db.sync()
    db.close()
    return n


def image_folder_records(root):
    """``root/<class>/<file>`` -> (raw encoded bytes, class index), classes in sorted order."""
    classes = sorted(d for d in os.listdir(root) if os.path.isdir(os.path.join(root, d)))
    for ci, c in enumerate(classes):
        for name in sorted(os.listdir(os.path.join(root, c))):
            with open(os.path.join(root, c, name), "rb") as f:
                yield f.read(), ci


def libsvm_records(path, n_features=None):
    """LIBSVM text lines ``label idx:val ...`` -> (dense float32 features, label in {0, 1})."""
    rows = []
    with open(path) as f:
        for line in f:
            parts = line.split()
            if not parts:
                continue
            idx = np.array([int(p.split(":")[0]) for p in parts[1:]], dtype=np.int64)
            val = np.array([float(p.split(":")[1]) for p in parts[1:]], dtype=np.float32)
            rows.append((float(parts[0]), idx, val))
    d = n_features or max(int(r[1].max()) for r in rows if len(r[1]))
    for label, idx, val in rows:
        x = np.zeros(d, dtype=np.float32)
        x[idx - 1] = val
        yield x, int(label > 0)


def main(argv=None):
    p = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    p.add_argument("--folder", default=None, help="ImageFolder-style root")
    p.add_argument("--split", default="train")
    p.add_argument("--libsvm", default=None, help="LIBSVM text file (epsilon, rcv1)")
    p.add_argument("--n_features", type=int, default=None)
    p.add_argument("--out", required=True)
    a = p.parse_args(argv)
    if a.folder:
        n = write_records(a.out, image_folder_records(os.path.join(a.folder, a.split)))
    elif a.libsvm:
        n = write_records(a.out, libsvm_records(a.libsvm, a.n_features))
    else:
        p.error("give --folder or --libsvm")
    print(f"wrote {n} records to {a.out}")


if __name__ == "__main__":
    main()
