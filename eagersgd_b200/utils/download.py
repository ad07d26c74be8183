"""Fetching data-set and model files: download into a cache folder, skip what is already there, unpack archives.

Counterpart of deep500/utils/download.py (``real_download``, ``unzip``, ``is_file_in_dir``) and of the
``download_*_and_get_file_paths`` helpers of its data sets (deep500/datasets/mnist.py:13-48, cifar.py).  Any URL
scheme ``urllib`` knows works — ``https://`` where there is a network, ``file://`` for a mirror on disk (what the
tests use: there is no network on the build machines).  A failed transfer leaves no partial file behind.
"""
from __future__ import annotations

import gzip
import hashlib
import os
import shutil
import tarfile
import tempfile
import urllib.request
import zipfile
from typing import Callable, Dict, Optional, Sequence

MNIST_FILES = {"train_images": "train-images-idx3-ubyte.gz", "train_labels": "train-labels-idx1-ubyte.gz",
               "test_images": "t10k-images-idx3-ubyte.gz", "test_labels": "t10k-labels-idx1-ubyte.gz"}
MNIST_URL = "http://yann.lecun.com/exdb/mnist/"
FASHION_MNIST_URL = "http://fashion-mnist.s3-website.eu-central-1.amazonaws.com/"
CIFAR10_URL, CIFAR10_FILE = "https://www.cs.toronto.edu/~kriz/", "cifar-10-python.tar.gz"   # what load_cifar10 reads


def default_cache_dir(sub_folder: str = "") -> str:
    base = os.environ.get("ESGD_DATA_DIR") or os.path.join(tempfile.gettempdir(), "eagersgd_data")
    return os.path.join(base, sub_folder) if sub_folder else base


def is_file_in_dir(directory: str, file_name: str) -> bool:
    return os.path.isfile(os.path.join(directory, file_name))


def sha256_of(path: str) -> str:
    h = hashlib.sha256()
    with open(path, "rb") as f:
        for chunk in iter(lambda: f.read(1 << 20), b""):
            h.update(chunk)
    return h.hexdigest()


def real_download(base_url: str, filenames: Sequence[str], sub_folder: str = "", output_dir: str = "",
                  sha256: Optional[Dict[str, str]] = None, progress: Optional[Callable[[str, int, int], None]] = None,
                  timeout: float = 60.0) -> Dict[str, str]:
    """Download ``base_url + name`` for every name into ``output_dir`` (default: the cache folder) / ``sub_folder``;
    files that are already there are kept.  ``sha256``: expected digests by file name (a mismatch raises and the file
    is removed).  ``progress(name, bytes_done, bytes_total)`` is called as data arrives.  Returns name -> local path."""
    folder = os.path.join(output_dir, sub_folder) if output_dir else default_cache_dir(sub_folder)
    os.makedirs(folder, exist_ok=True)
    if not base_url.endswith(("/", "=")):
        base_url += "/"
    out = {}
    for name in filenames:
        dst = os.path.join(folder, os.path.basename(name))
        if not os.path.isfile(dst):
            tmp = dst + ".part"
            try:
                with urllib.request.urlopen(base_url + name, timeout=timeout) as r, open(tmp, "wb") as f:
                    total = int(r.headers.get("Content-Length") or 0) if hasattr(r, "headers") else 0
                    done = 0
                    for chunk in iter(lambda: r.read(1 << 20), b""):
                        f.write(chunk)
                        done += len(chunk)
                        if progress is not None:
                            progress(name, done, total)
                os.replace(tmp, dst)
            except Exception as e:
                if os.path.exists(tmp):
                    os.remove(tmp)
                raise IOError("could not fetch %s: %s" % (base_url + name, e)) from e
        if sha256 and name in sha256 and sha256_of(dst) != sha256[name]:
            os.remove(dst)
            raise IOError("%s: checksum mismatch, file removed" % name)
        out[name] = dst
    return out


def unpack(local_file: str, into: Optional[str] = None) -> str:
    """Unpack a .zip, .tar, .tar.gz / .tgz or .gz file next to itself (or ``into``); returns the folder (the file
    for a plain .gz).  Already unpacked content is left alone."""
    into = into or os.path.dirname(local_file)
    if local_file.endswith(".zip"):
        with zipfile.ZipFile(local_file) as z:
            z.extractall(into)
        return into
    if local_file.endswith((".tar", ".tar.gz", ".tgz")):
        with tarfile.open(local_file) as t:
            base = os.path.realpath(into)
            for m in t.getmembers():                       # nothing may land outside the target folder
                if not os.path.realpath(os.path.join(into, m.name)).startswith(base + os.sep):
                    raise IOError("archive member escapes the target folder: %s" % m.name)
            t.extractall(into)
        return into
    if local_file.endswith(".gz"):
        dst = os.path.join(into, os.path.basename(local_file)[:-3])
        if not os.path.isfile(dst):
            with gzip.open(local_file, "rb") as src, open(dst + ".part", "wb") as f:
                shutil.copyfileobj(src, f)
            os.replace(dst + ".part", dst)
        return dst
    raise ValueError("do not know how to unpack %s" % local_file)


unzip = unpack


def download_mnist_and_get_file_paths(folder: str = "", base_url: str = MNIST_URL) -> Dict[str, str]:
    """The four MNIST files by role (``train_images`` ...), fetched if they are not in ``folder`` yet."""
    got = real_download(base_url, list(MNIST_FILES.values()), "mnist", folder)
    return {role: got[name] for role, name in MNIST_FILES.items()}


def download_fashion_mnist_and_get_file_paths(folder: str = "", base_url: str = FASHION_MNIST_URL) -> Dict[str, str]:
    got = real_download(base_url, list(MNIST_FILES.values()), "fashion_mnist", folder)
    return {role: got[name] for role, name in MNIST_FILES.items()}


def download_cifar10_and_get_folder(folder: str = "", base_url: str = CIFAR10_URL) -> str:
    """The CIFAR-10 python batches, fetched and unpacked; returns the folder that holds ``data_batch_1`` ...
    ``test_batch`` (the argument of ``data.dataset.load_cifar10``)."""
    got = real_download(base_url, [CIFAR10_FILE], "cifar10", folder)
    root = unpack(got[CIFAR10_FILE])
    sub = os.path.join(root, "cifar-10-batches-py")
    return sub if os.path.isdir(sub) else root
