"""Augmentation toolkit, record packing / reading, feature datasets and pretrained embeddings."""
import os

import numpy as np
import torch

from chocosgd_b200.data import augment as A
from chocosgd_b200.data import serialize
from chocosgd_b200.data.embeddings import find_vector_file, load_vectors
from chocosgd_b200.data.lmdb_dataset import LMDBImageDataset, define_epsilon_or_rcv1_folder


def test_random_crop_windows_are_slices_of_the_padded_image():
    x = torch.arange(2 * 1 * 6 * 6, dtype=torch.float32).view(2, 1, 6, 6)
    out = A.RandomCrop(4, padding=1)(x, torch.Generator().manual_seed(3))
    padded = torch.nn.functional.pad(x, [1] * 4)
    for b in range(2):
        hits = [(t, l) for t in range(5) for l in range(5) if torch.equal(padded[b, :, t:t + 4, l:l + 4], out[b])]
        assert hits, "crop is not a window of the padded image"


def test_flip_and_recipes_shapes_and_determinism():
    g1, g2 = torch.Generator().manual_seed(5), torch.Generator().manual_seed(5)
    x = torch.rand(6, 3, 64, 80)
    t = A.get_transform("imagenet", input_size=32, color_process=True)
    a, b = t(x, g1), t(x, g2)
    assert a.shape == (6, 3, 32, 32) and torch.equal(a, b)
    assert A.get_transform("imagenet", augment=False)(torch.rand(2, 3, 300, 280)).shape == (2, 3, 224, 224)
    assert A.get_transform("cifar10")(torch.rand(2, 3, 32, 32)).shape == (2, 3, 32, 32)
    assert A.get_transform("mnist")(torch.rand(2, 1, 28, 28)).shape == (2, 1, 28, 28)
    flipped = A.RandomHorizontalFlip()(x, torch.Generator().manual_seed(0))
    for i in range(6):
        assert torch.equal(flipped[i], x[i]) or torch.equal(flipped[i], x[i].flip(-1))


def test_colour_transforms_match_their_definitions():
    x = torch.rand(3, 3, 8, 8)
    gray = A.grayscale(x)
    torch.testing.assert_close(gray[:, 0], 0.299 * x[:, 0] + 0.587 * x[:, 1] + 0.114 * x[:, 2])
    assert torch.equal(A.Saturation(0.0)(x), x) and torch.equal(A.Lighting(0.0)(x), x)
    lit = A.Lighting(0.1)(x, torch.Generator().manual_seed(1))
    shift = (lit - x)
    assert torch.allclose(shift, shift[:, :, :1, :1].expand_as(shift), atol=1e-6)   # one RGB offset per image
    n = A.Normalize([0.5, 0.5, 0.5], [0.25, 0.25, 0.25])(x)
    torch.testing.assert_close(n, (x - 0.5) / 0.25)


def test_record_file_round_trip_and_feature_dataset(tmp_path):
    path = str(tmp_path / "epsilon_train.lmdb")   # falls back to the record file where lmdb is missing
    feats = [np.random.RandomState(i).rand(12).astype(np.float32) for i in range(7)]
    n = serialize.write_records(path, ((f, i % 2) for i, f in enumerate(feats)), use_lmdb=False)
    assert n == 7
    ds = define_epsilon_or_rcv1_folder(path)
    assert len(ds) == 7
    x, y = ds[4]
    np.testing.assert_array_equal(x.numpy(), feats[4])
    assert y == 0


def test_libsvm_parser_and_image_records(tmp_path):
    svm = tmp_path / "tiny.svm"
    svm.write_text("+1 1:0.5 3:2\n-1 2:1.5\n")
    recs = list(serialize.libsvm_records(str(svm), n_features=4))
    np.testing.assert_array_equal(recs[0][0], np.array([0.5, 0, 2, 0], dtype=np.float32))
    assert [r[1] for r in recs] == [1, 0]
    from PIL import Image

    root = tmp_path / "imgs" / "train"
    for c in ("a", "b"):
        os.makedirs(root / c)
        Image.fromarray((np.random.rand(8, 8, 3) * 255).astype(np.uint8)).save(root / c / "0.png")
    out = str(tmp_path / "train.rec")
    assert serialize.write_records(out, serialize.image_folder_records(str(root))) == 2
    ds = LMDBImageDataset(out, "imagenet", transform=A.per_sample(A.get_transform("cifar10", input_size=8, augment=False)))
    img, label = ds[1]
    assert img.shape == (3, 8, 8) and label == 1


def test_pretrained_vectors_align_with_the_dictionary(tmp_path):
    (tmp_path / "glove.test.txt").write_text("the 1 2 3\ncat 4 5 6\n")
    f = find_vector_file(str(tmp_path))
    w, found = load_vectors(f, {"<eos>": 0, "cat": 1, "the": 2})
    assert found == 2 and w.shape == (3, 3)
    assert w[1].tolist() == [4, 5, 6] and w[2].tolist() == [1, 2, 3] and w[0].abs().max() <= 0.1
