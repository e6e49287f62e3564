"""Directory helpers (``dl_code/pcode/utils/op_paths.py``)."""
import os
import shutil


def get_current_path(conf, rank):
    paths_from_previous = conf.resume.split(",")
    return paths_from_previous[rank] if len(paths_from_previous) > 1 else conf.resume


def list_files(root_path):
    dirs = os.listdir(root_path)
    return [os.path.join(root_path, path) for path in dirs]


def build_dir(path, force=False):
    if os.path.exists(path) and force:
        shutil.rmtree(path)
    os.makedirs(path, exist_ok=True)


def build_dirs(path):
    try:
        os.makedirs(path, exist_ok=True)
    except OSError as e:
        print(" encounter error: {}".format(e))


def remove_folder(path):
    try:
        shutil.rmtree(path)
    except OSError as e:
        print(" encounter error: {}".format(e))
