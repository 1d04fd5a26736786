"""Vision datasets (``python/mxnet/gluon/data/vision/datasets.py``).  Files are read from ``root``;
they are fetched only when absent (there is no bundled data)."""
import gzip
import os
import pickle
import struct
import tarfile
import warnings

import numpy as np

from .... import env
from ..dataset import Dataset, RecordFileDataset

__all__ = ['MNIST', 'FashionMNIST', 'CIFAR10', 'CIFAR100', 'ImageRecordDataset', 'ImageFolderDataset', 'ImageListDataset']


def _wrap(a):
    from ....util import is_np_array
    if is_np_array():
        from .... import numpy as mnp
        return mnp.array(a, dtype=a.dtype)
    from .... import ndarray as nd
    return nd.array(a, dtype=a.dtype)


class _DownloadedDataset(Dataset):
    def __init__(self, root, transform):
        self._transform = transform
        self._data = self._label = None
        self._root = os.path.expanduser(root)
        os.makedirs(self._root, exist_ok=True)
        self._get_data()

    def __getitem__(self, idx):
        if self._transform is not None:
            return self._transform(_wrap(self._data[idx]), self._label[idx])
        return _wrap(self._data[idx]), self._label[idx]

    def __len__(self):
        return len(self._label)

    def _fetch(self, name, url):
        path = os.path.join(self._root, name)
        if not os.path.exists(path):
            from ...utils import download
            download(url, path=path)
        return path


class MNIST(_DownloadedDataset):
    _base = 'gluon/dataset/mnist/'
    _files = {True: ('train-images-idx3-ubyte.gz', 'train-labels-idx1-ubyte.gz'),
              False: ('t10k-images-idx3-ubyte.gz', 't10k-labels-idx1-ubyte.gz')}

    def __init__(self, root=os.path.join(env.get('MXNET_HOME'), 'datasets', 'mnist'), train=True, transform=None):
        self._train = train
        super().__init__(root, transform)

    def _get_data(self):
        data_file, label_file = self._files[self._train]
        repo = env.get('MXNET_GLUON_REPO')
        dpath = self._fetch(data_file, repo + self._base + data_file)
        lpath = self._fetch(label_file, repo + self._base + label_file)
        with gzip.open(lpath, 'rb') as fin:
            struct.unpack('>II', fin.read(8))
            label = np.frombuffer(fin.read(), dtype=np.uint8).astype(np.int32)
        with gzip.open(dpath, 'rb') as fin:
            struct.unpack('>IIII', fin.read(16))
            data = np.frombuffer(fin.read(), dtype=np.uint8).reshape(len(label), 28, 28, 1)
        self._data, self._label = data, label


class FashionMNIST(MNIST):
    _base = 'gluon/dataset/fashion-mnist/'

    def __init__(self, root=os.path.join(env.get('MXNET_HOME'), 'datasets', 'fashion-mnist'), train=True, transform=None):
        super().__init__(root, train, transform)


class CIFAR10(_DownloadedDataset):
    def __init__(self, root=os.path.join(env.get('MXNET_HOME'), 'datasets', 'cifar10'), train=True, transform=None):
        self._train = train
        self._archive = 'cifar-10-binary.tar.gz'
        self._train_files = ['data_batch_%d.bin' % i for i in range(1, 6)]
        self._test_files = ['test_batch.bin']
        self._namespace = 'cifar10'
        super().__init__(root, transform)

    def _read_batch(self, filename):
        with open(filename, 'rb') as fin:
            data = np.frombuffer(fin.read(), dtype=np.uint8).reshape(-1, 3072 + 1)
        return data[:, 1:].reshape(-1, 3, 32, 32).transpose(0, 2, 3, 1), data[:, 0].astype(np.int32)

    def _get_data(self):
        files = self._train_files if self._train else self._test_files
        if not all(os.path.exists(os.path.join(self._root, f)) for f in files):
            arc = self._fetch(self._archive, env.get('MXNET_GLUON_REPO') + 'gluon/dataset/%s/%s' % (self._namespace, self._archive))
            with tarfile.open(arc) as tar:
                for m in tar.getmembers():
                    if m.isfile():
                        m.name = os.path.basename(m.name)
                        tar.extract(m, self._root)
        data, label = zip(*(self._read_batch(os.path.join(self._root, f)) for f in files))
        self._data, self._label = np.concatenate(data), np.concatenate(label)


class CIFAR100(CIFAR10):
    def __init__(self, root=os.path.join(env.get('MXNET_HOME'), 'datasets', 'cifar100'), fine_label=False, train=True,
                 transform=None):
        self._fine_label = fine_label
        self._train = train
        self._archive = 'cifar-100-binary.tar.gz'
        self._train_files, self._test_files = ['train.bin'], ['test.bin']
        self._namespace = 'cifar100'
        _DownloadedDataset.__init__(self, root, transform)

    def _read_batch(self, filename):
        with open(filename, 'rb') as fin:
            data = np.frombuffer(fin.read(), dtype=np.uint8).reshape(-1, 3072 + 2)
        return data[:, 2:].reshape(-1, 3, 32, 32).transpose(0, 2, 3, 1), data[:, 0 + self._fine_label].astype(np.int32)


class ImageRecordDataset(RecordFileDataset):
    def __init__(self, filename, flag=1, transform=None):
        super().__init__(filename)
        self._flag, self._transform = flag, transform

    def __getitem__(self, idx):
        from .... import recordio, image
        record = super().__getitem__(idx)
        header, img = recordio.unpack(record)
        img = image.imdecode(img, self._flag)
        if self._transform is not None:
            return self._transform(img, header.label)
        return img, header.label


class ImageFolderDataset(Dataset):
    def __init__(self, root, flag=1, transform=None):
        self._root = os.path.expanduser(root)
        self._flag, self._transform = flag, transform
        self._exts = ['.jpg', '.jpeg', '.png']
        self._list_images(self._root)

    def _list_images(self, root):
        self.synsets, self.items = [], []
        for folder in sorted(os.listdir(root)):
            path = os.path.join(root, folder)
            if not os.path.isdir(path):
                warnings.warn('Ignoring %s, which is not a directory.' % path, stacklevel=3)
                continue
            label = len(self.synsets)
            self.synsets.append(folder)
            for filename in sorted(os.listdir(path)):
                fpath = os.path.join(path, filename)
                if os.path.splitext(filename)[1].lower() not in self._exts:
                    warnings.warn('Ignoring %s of type %s. Only support %s' % (filename, os.path.splitext(filename)[1],
                                                                               ', '.join(self._exts)))
                    continue
                self.items.append((fpath, label))

    def __getitem__(self, idx):
        from .... import image
        img = image.imread(self.items[idx][0], self._flag)
        label = self.items[idx][1]
        if self._transform is not None:
            return self._transform(img, label)
        return img, label

    def __len__(self):
        return len(self.items)


class ImageListDataset(Dataset):
    def __init__(self, root='.', imglist=None, flag=1):
        self._root, self._flag = os.path.expanduser(root), flag
        self.items = []
        if isinstance(imglist, str):
            with open(os.path.join(self._root, imglist)) as f:
                for line in f:
                    parts = line.strip().split('\t')
                    label = [float(i) for i in parts[1:-1]]
                    self.items.append((os.path.join(self._root, parts[-1]), label[0] if len(label) == 1 else label))
        else:
            for item in imglist or []:
                label = item[:-1] if len(item) > 2 else item[0]
                self.items.append((os.path.join(self._root, item[-1]), label))

    def __getitem__(self, idx):
        from .... import image
        return image.imread(self.items[idx][0], self._flag), self.items[idx][1]

    def __len__(self):
        return len(self.items)
