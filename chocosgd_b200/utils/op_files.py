"""Small file readers / writers (``dl_code/pcode/utils/op_files.py``)."""
import json
import pickle


def read_text_withoutsplit(path):
    with open(path, "r") as f:
        return f.read()


def read_txt(path):
    with open(path, "r") as f:
        return f.read().splitlines()


def write_txt(data, out_path, type="w"):
    with open(out_path, type) as f:
        f.write(data)


def load_pickle(path):
    with open(path, "rb") as handle:
        return pickle.load(handle)


def write_pickle(data, path):
    with open(path, "wb") as handle:
        pickle.dump(data, handle, protocol=pickle.HIGHEST_PROTOCOL)


def read_json(path):
    with open(path, "r") as f:
        return json.load(f)


def is_jsonable(x):
    try:
        json.dumps(x)
        return True
    except (TypeError, OverflowError):
        return False
