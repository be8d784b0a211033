"""Vision datasets (MNIST / CIFAR with synthetic fallbacks, ImageFolder / DatasetFolder), image IO and the transform set.

Reference parity: ferrotorch-vision/src/{mnist.rs:58, cifar.rs:81-197, folder.rs:50-156, io.rs:43-135} and the 16 transforms
(center_crop ... vision_normalize).
"""
from __future__ import annotations

import enum
import gzip
import math
import threading
import os
import pickle
import struct
from pathlib import Path
from dataclasses import dataclass
from typing import Callable, List, NamedTuple, Optional, Sequence, Tuple

import numpy as np
import torch
import torch.nn.functional as F

from ..data import Dataset
from ..errors import InvalidArgument
from ..nn import resample as _resample


# -- image IO (PNG/JPEG via Pillow, PPM natively) ---------------------------------------------------------------------------------------
def read_image(path) -> torch.Tensor:
    """``[C,H,W]`` uint8 tensor."""
    p = str(path)
    if p.lower().endswith((".ppm", ".pgm")):
        with open(p, "rb") as f:
            magic = f.readline().strip()
            line = f.readline()
            while line.startswith(b"#"):
                line = f.readline()
            w, h = map(int, line.split())
            maxv = int(f.readline())
            c = 3 if magic == b"P6" else 1
            data = np.frombuffer(f.read(w * h * c), dtype=np.uint8).reshape(h, w, c)
        return torch.from_numpy(data.copy()).permute(2, 0, 1)
    from PIL import Image
    a = np.asarray(Image.open(p).convert("RGB"))
    return torch.from_numpy(a.copy()).permute(2, 0, 1)


def write_image(path, img: torch.Tensor) -> None:
    a = img.detach().cpu()
    if a.is_floating_point():
        a = (a.clamp(0, 1) * 255).round().to(torch.uint8)
    a = a.permute(1, 2, 0).contiguous().numpy()
    p = str(path)
    if p.lower().endswith(".ppm"):
        with open(p, "wb") as f:
            f.write(f"P6\n{a.shape[1]} {a.shape[0]}\n255\n".encode())
            f.write(a.tobytes())
        return
    from PIL import Image
    Image.fromarray(a.squeeze(-1) if a.shape[-1] == 1 else a).save(p)


@dataclass
class RawImage:
    """Decoded 8-bit image in row-major ``[H, W, C]`` byte order (ferrotorch-vision/src/io.rs:23)."""
    data: bytes
    width: int
    height: int
    channels: int


def _raw(t: torch.Tensor) -> RawImage:                       # [C, H, W] uint8
    return RawImage(t.permute(1, 2, 0).contiguous().numpy().tobytes(), int(t.shape[2]), int(t.shape[1]), int(t.shape[0]))


def read_image_raw(path) -> RawImage:
    """RGB bytes of an image file; the reference's ``read_image`` (io.rs:41; :func:`read_image` here returns the ``[C, H, W]`` tensor directly)."""
    try:
        return _raw(read_image(path))
    except Exception as e:
        raise InvalidArgument(f"failed to read image '{path}': {e}") from None


def read_image_rgba(path) -> RawImage:
    """RGBA bytes; images without an alpha channel get alpha 255 (io.rs:62)."""
    try:
        from PIL import Image
        a = np.asarray(Image.open(str(path)).convert("RGBA"))
    except Exception as e:
        raise InvalidArgument(f"failed to read image '{path}': {e}") from None
    return RawImage(a.tobytes(), a.shape[1], a.shape[0], 4)


def raw_image_to_tensor(raw: RawImage, dtype=torch.float32) -> torch.Tensor:
    """``[C, H, W]`` float tensor in [0, 1] (io.rs:106)."""
    n = raw.height * raw.width * raw.channels
    if len(raw.data) != n:
        raise InvalidArgument(f"raw_image_to_tensor: {len(raw.data)} bytes for {raw.height}x{raw.width}x{raw.channels}")
    a = torch.frombuffer(bytearray(raw.data), dtype=torch.uint8).view(raw.height, raw.width, raw.channels)
    return a.permute(2, 0, 1).to(dtype).div(255).contiguous()


def read_image_as_tensor(path, dtype=torch.float32) -> torch.Tensor:
    return raw_image_to_tensor(read_image_raw(path), dtype)


def tensor_to_raw_image(t: torch.Tensor) -> RawImage:
    """``[C, H, W]`` with 3 or 4 channels, values clamped to [0, 1], times 255, rounded (io.rs:203)."""
    if t.dim() != 3:
        raise InvalidArgument(f"tensor_to_raw_image: expected 3-D tensor [C, H, W], got shape {list(t.shape)}")
    if t.shape[0] not in (3, 4):
        raise InvalidArgument(f"tensor_to_raw_image: expected 3 or 4 channels, got {t.shape[0]}")
    return _raw((t.detach().cpu().double().clamp(0, 1) * 255).round().to(torch.uint8))


def write_raw_image(path, raw: RawImage) -> None:
    a = torch.frombuffer(bytearray(raw.data), dtype=torch.uint8).view(raw.height, raw.width, raw.channels).permute(2, 0, 1)
    try:
        write_image(path, a)
    except Exception as e:
        raise InvalidArgument(f"failed to write image '{path}': {e}") from None


def write_tensor_as_image(path, t: torch.Tensor) -> None:
    write_raw_image(path, tensor_to_raw_image(t))


class Split(enum.Enum):
    """Which half of a dataset to load (ferrotorch-vision/src/datasets/mnist.rs:43)."""
    Train = "train"
    Test = "test"


class MnistSample(NamedTuple):
    """``(image [1, 28, 28], label)`` (datasets/mnist.rs:34); unpacks like the plain tuple it is."""
    image: torch.Tensor
    label: int


class CifarSample(NamedTuple):
    """``(image [3, 32, 32], label)`` (datasets/cifar.rs:53)."""
    image: torch.Tensor
    label: int


IMAGENET_MEAN = (0.485, 0.456, 0.406)                        # ferrotorch-vision/src/transforms/mod.rs:38-41
IMAGENET_STD = (0.229, 0.224, 0.225)


# -- datasets ---------------------------------------------------------------------------------------------------------------------------
class Mnist(Dataset):
    """MNIST from the IDX files under ``root`` or a deterministic synthetic stand-in (class-dependent blob patterns)."""

    def __init__(self, images: torch.Tensor, labels: torch.Tensor, transform: Optional[Callable] = None):
        self.images, self.labels, self.transform = images, labels, transform

    @staticmethod
    def from_dir(root, train=True, transform=None) -> "Mnist":
        train = train is Split.Train if isinstance(train, Split) else bool(train)
        pre = "train" if train else "t10k"

        def idx(name):
            p = Path(root) / name
            op = gzip.open if not p.exists() and (p.with_suffix(p.suffix + ".gz")).exists() else open
            with op(p if p.exists() else str(p) + ".gz", "rb") as f:
                magic, n = struct.unpack(">II", f.read(8))
                if magic == 2051:
                    r, c = struct.unpack(">II", f.read(8))
                    return np.frombuffer(f.read(), dtype=np.uint8).reshape(n, r, c)
                return np.frombuffer(f.read(), dtype=np.uint8)
        return Mnist(torch.from_numpy(idx(f"{pre}-images-idx3-ubyte").copy()).float().div(255).unsqueeze(1),
                     torch.from_numpy(idx(f"{pre}-labels-idx1-ubyte").copy()).long(), transform)

    @staticmethod
    def synthetic(n: int = 1024, seed: int = 0, transform=None) -> "Mnist":
        g = torch.Generator().manual_seed(seed)
        labels = torch.randint(0, 10, (n,), generator=g)
        yy, xx = torch.meshgrid(torch.arange(28.), torch.arange(28.), indexing="ij")
        imgs = torch.zeros(n, 1, 28, 28)
        for c in range(10):
            cx, cy = 6 + 4 * (c % 5), 8 + 10 * (c // 5)
            pat = torch.exp(-((xx - cx) ** 2 + (yy - cy) ** 2) / 18.0)
            imgs[labels == c, 0] = pat
        imgs += 0.1 * torch.randn(n, 1, 28, 28, generator=g)
        return Mnist(imgs.clamp(0, 1), labels, transform)

    def __len__(self):
        return len(self.labels)

    def __getitem__(self, i):
        x = self.images[i]
        return MnistSample((self.transform(x) if self.transform else x), self.labels[i])


class Cifar10(Dataset):
    classes = 10

    def __init__(self, images: torch.Tensor, labels: torch.Tensor, transform=None):
        self.images, self.labels, self.transform = images, labels, transform

    @classmethod
    def from_dir(cls, root, train=True, transform=None):
        train = train is Split.Train if isinstance(train, Split) else bool(train)
        files = [f"data_batch_{i}" for i in range(1, 6)] if train else ["test_batch"]
        if cls.classes == 100:
            files = ["train"] if train else ["test"]
        xs, ys = [], []
        for fn in files:
            with open(Path(root) / fn, "rb") as f:
                d = pickle.load(f, encoding="bytes")
            xs.append(np.asarray(d[b"data"], dtype=np.uint8).reshape(-1, 3, 32, 32))
            ys += list(d[b"labels"] if b"labels" in d else d[b"fine_labels"])
        return cls(torch.from_numpy(np.concatenate(xs)).float().div(255), torch.tensor(ys), transform)

    @classmethod
    def synthetic(cls, n: int = 1024, seed: int = 0, transform=None):
        g = torch.Generator().manual_seed(seed)
        labels = torch.randint(0, cls.classes, (n,), generator=g)
        base = torch.rand(cls.classes, 3, 1, 1, generator=g)
        imgs = (base[labels] + 0.15 * torch.randn(n, 3, 32, 32, generator=g)).clamp(0, 1)
        return cls(imgs, labels, transform)

    def __len__(self):
        return len(self.labels)

    def __getitem__(self, i):
        x = self.images[i]
        return CifarSample((self.transform(x) if self.transform else x), self.labels[i])


class Cifar100(Cifar10):
    classes = 100


class DatasetFolder(Dataset):
    """``root/<class>/<file>`` layout; ``loader(path)`` turns a file into a sample."""

    def __init__(self, root, loader: Callable, extensions: Sequence[str], transform=None):
        self.root, self.loader, self.transform = Path(root), loader, transform
        self.classes = sorted(d.name for d in self.root.iterdir() if d.is_dir())
        self.class_to_idx = {c: i for i, c in enumerate(self.classes)}
        self.samples: List[Tuple[Path, int]] = []
        for c in self.classes:
            for f in sorted((self.root / c).rglob("*")):
                if f.suffix.lower() in extensions:
                    self.samples.append((f, self.class_to_idx[c]))
        if not self.samples:
            raise InvalidArgument(f"no files with extensions {list(extensions)} under {root}")

    def __len__(self):
        return len(self.samples)

    def __getitem__(self, i):
        p, y = self.samples[i]
        x = self.loader(p)
        return (self.transform(x) if self.transform else x), y


class ImageFolder(DatasetFolder):
    def __init__(self, root, transform=None):
        super().__init__(root, read_image, (".png", ".jpg", ".jpeg", ".ppm", ".bmp"), transform)


# -- transforms (operate on [C,H,W] tensors) ----------------------------------------------------------------------------------------------------
# -- random source of the augmentation transforms ---------------------------------------------------------------------------------------
class _VisionRng:
    """Counter-based splitmix64 stream with its own seed (default 42), separate from the tensor RNGs so that augmentation can be replayed on
    its own: draw number n after ``vision_manual_seed(s)`` is a pure function of (s, n), as in
    ferrotorch-vision/src/transforms/rng.rs:17-47 (same mixing constants, same mapping to [0, 1])."""
    _M = (1 << 64) - 1

    def __init__(self):
        self.seed, self.draw = 42, 0
        self._lock = threading.Lock()

    def manual_seed(self, seed: int) -> None:
        with self._lock:
            self.seed, self.draw = int(seed) & self._M, 0

    def random(self) -> float:
        with self._lock:
            d = self.draw
            self.draw += 1
        z = (self.seed + d * 0x9E3779B97F4A7C15) & self._M
        z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & self._M
        z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & self._M
        z ^= z >> 31
        return z / float(self._M)

    def uniform(self, lo: float, hi: float) -> float:
        return lo + (hi - lo) * self.random()

    def randint(self, upper: int) -> int:                # rng.rs:45-47
        return int(self.random() * upper) % upper

    def generator(self) -> torch.Generator:
        """A torch generator keyed by the next draw, for transforms that need whole random tensors (noise, displacement fields)."""
        return torch.Generator().manual_seed(int(self.random() * (1 << 62)))


_vision_rng = _VisionRng()


def vision_manual_seed(seed: int) -> None:
    """Seed the augmentation stream (ferrotorch-vision/src/transforms/rng.rs:24-30)."""
    _vision_rng.manual_seed(seed)


class Compose:
    def __init__(self, ts):
        self.ts = list(ts)

    def __call__(self, x):
        for t in self.ts:
            x = t(x)
        return x


class ToTensor:
    def __call__(self, x):
        if isinstance(x, np.ndarray):
            x = torch.from_numpy(x)
            if x.dim() == 3 and x.shape[-1] in (1, 3, 4):
                x = x.permute(2, 0, 1)
        return x.float().div(255) if x.dtype == torch.uint8 else x.float()


class VisionToTensor:
    """``[H, W, C]`` image with values in 0..255 (any dtype) -> float ``[C, H, W]`` in 0..1: always transposes and always divides by 255, as
    ferrotorch-vision/src/transforms/to_tensor.rs:24-57 does (:class:`ToTensor` only rescales 8-bit input)."""

    def __call__(self, x):
        if isinstance(x, np.ndarray):
            x = torch.from_numpy(x)
        if x.dim() != 3:
            raise InvalidArgument(f"VisionToTensor: expected 3-D tensor [H, W, C], got shape {list(x.shape)}")
        return x.permute(2, 0, 1).float().div(255).contiguous()


class VisionNormalize:
    def __init__(self, mean, std):
        self.mean, self.std = torch.tensor(mean).view(-1, 1, 1), torch.tensor(std).view(-1, 1, 1)

    def __call__(self, x):
        return (x - self.mean.to(x)) / self.std.to(x)


class Resize:
    """Resize a ``[C, H, W]`` image. The default is the reference's rule, nearest neighbour with source index ``floor(dst * in / out)``
    (ferrotorch-vision/src/transforms/resize.rs:44-52); ``mode="bilinear"`` / ``"bicubic"`` are extensions."""

    def __init__(self, size, mode="nearest"):
        self.size, self.mode = (size, size) if isinstance(size, int) else tuple(size), mode

    def __call__(self, x):
        return _resample.interpolate(x.unsqueeze(0).float(), self.size, mode=self.mode, align_corners=False if self.mode != "nearest" else None).squeeze(0)


class CenterCrop:
    def __init__(self, size):
        self.size = (size, size) if isinstance(size, int) else tuple(size)

    def __call__(self, x):
        h, w = x.shape[-2:]
        th, tw = self.size
        if th > h or tw > w:               # ferrotorch-vision/src/transforms/center_crop.rs:43-49
            raise InvalidArgument(f"CenterCrop: crop size ({th}x{tw}) is larger than input spatial size ({h}x{w})")
        i, j = (h - th) // 2, (w - tw) // 2
        return x[..., i: i + th, j: j + tw]


class RandomCrop:
    def __init__(self, size, padding: int = 0):
        self.size, self.padding = (size, size) if isinstance(size, int) else tuple(size), padding

    def __call__(self, x):
        if self.padding:
            x = F.pad(x, [self.padding] * 4)
        h, w = x.shape[-2:]
        th, tw = self.size
        i, j = _vision_rng.randint(h - th + 1), _vision_rng.randint(w - tw + 1)
        return x[..., i: i + th, j: j + tw]


class RandomHorizontalFlip:
    def __init__(self, p=0.5):
        self.p = p

    def __call__(self, x):
        return x.flip(-1) if _vision_rng.random() < self.p else x


class RandomVerticalFlip(RandomHorizontalFlip):
    def __call__(self, x):
        return x.flip(-2) if _vision_rng.random() < self.p else x


class RandomResizedCrop:
    def __init__(self, size, scale=(0.08, 1.0), ratio=(3 / 4, 4 / 3)):
        self.size, self.scale, self.ratio = (size, size) if isinstance(size, int) else tuple(size), scale, ratio

    def __call__(self, x):
        h, w = x.shape[-2:]
        for _ in range(10):
            area = h * w * _vision_rng.uniform(*self.scale)
            r = math.exp(_vision_rng.uniform(math.log(self.ratio[0]), math.log(self.ratio[1])))
            cw, ch = int(round(math.sqrt(area * r))), int(round(math.sqrt(area / r)))
            if 0 < cw <= w and 0 < ch <= h:
                i, j = _vision_rng.randint(h - ch + 1), _vision_rng.randint(w - cw + 1)
                return Resize(self.size)(x[..., i: i + ch, j: j + cw])
        return Resize(self.size)(CenterCrop(min(h, w))(x))


class RandomRotation:
    def __init__(self, degrees: float):
        self.degrees = degrees

    def __call__(self, x):
        a = math.radians(_vision_rng.uniform(-self.degrees, self.degrees))
        theta = torch.tensor([[math.cos(a), -math.sin(a), 0.0], [math.sin(a), math.cos(a), 0.0]]).unsqueeze(0)
        grid = _resample.affine_grid(theta, [1, *x.shape], align_corners=False)
        return _resample.grid_sample(x.unsqueeze(0).float(), grid, align_corners=False).squeeze(0)


class ColorJitter:
    def __init__(self, brightness=0.0, contrast=0.0, saturation=0.0):
        self.b, self.c, self.s = brightness, contrast, saturation

    def __call__(self, x):
        if self.b:
            x = x * _vision_rng.uniform(max(0, 1 - self.b), 1 + self.b)
        if self.c:
            m = x.mean()
            x = (x - m) * _vision_rng.uniform(max(0, 1 - self.c), 1 + self.c) + m
        if self.s and x.shape[0] == 3:
            g = (0.299 * x[0] + 0.587 * x[1] + 0.114 * x[2]).unsqueeze(0)
            x = (x - g) * _vision_rng.uniform(max(0, 1 - self.s), 1 + self.s) + g
        return x.clamp(0, 1)


class GaussianNoise:
    def __init__(self, std=0.05):
        self.std = std

    def __call__(self, x):
        return x + self.std * torch.randn(x.shape, generator=_vision_rng.generator()).to(x)


class RandomGaussianBlur:
    def __init__(self, kernel_size=3, sigma=(0.1, 2.0), p=0.5):
        self.k, self.sigma, self.p = kernel_size, sigma, p

    def __call__(self, x):
        if _vision_rng.random() >= self.p:
            return x
        s = _vision_rng.uniform(*self.sigma)
        ax = torch.arange(self.k, dtype=torch.float32) - (self.k - 1) / 2
        k1 = torch.exp(-ax ** 2 / (2 * s * s))
        k1 = k1 / k1.sum()
        c = x.shape[0]
        xx = F.conv2d(F.pad(x.unsqueeze(0).float(), [self.k // 2] * 4, mode="reflect"), k1.view(1, 1, 1, -1).repeat(c, 1, 1, 1), groups=c)
        return F.conv2d(xx, k1.view(1, 1, -1, 1).repeat(c, 1, 1, 1), groups=c).squeeze(0)


class RandomApply:
    def __init__(self, ts, p=0.5):
        self.t, self.p = Compose(ts), p

    def __call__(self, x):
        return self.t(x) if _vision_rng.random() < self.p else x


class RandomChoice:
    """Applies exactly one of the given transforms, picked uniformly (ferrotorch-vision/src/transforms/random_apply.rs:35-57)."""

    def __init__(self, ts):
        if not ts:
            raise InvalidArgument("RandomChoice: transforms list must not be empty")
        self.ts = list(ts)

    def __call__(self, x):
        return self.ts[min(int(_vision_rng.random() * len(self.ts)), len(self.ts) - 1)](x)


class ElasticTransform:
    def __init__(self, alpha=30.0, sigma=4.0):
        self.alpha, self.sigma = alpha, sigma

    def __call__(self, x):
        c, h, w = x.shape
        d = torch.randn(1, 2, h, w, generator=_vision_rng.generator())
        k = int(2 * round(3 * self.sigma) + 1)
        ax = torch.arange(k, dtype=torch.float32) - (k - 1) / 2
        g = torch.exp(-ax ** 2 / (2 * self.sigma ** 2))
        g = g / g.sum()
        d = F.conv2d(F.pad(d, [k // 2, k // 2, 0, 0], mode="reflect"), g.view(1, 1, 1, -1).repeat(2, 1, 1, 1), groups=2)
        d = F.conv2d(F.pad(d, [0, 0, k // 2, k // 2], mode="reflect"), g.view(1, 1, -1, 1).repeat(2, 1, 1, 1), groups=2) * self.alpha
        ys, xs = torch.meshgrid(torch.linspace(-1, 1, h), torch.linspace(-1, 1, w), indexing="ij")
        grid = torch.stack([xs + d[0, 0] * 2 / w, ys + d[0, 1] * 2 / h], -1).unsqueeze(0)
        return _resample.grid_sample(x.unsqueeze(0).float(), grid, align_corners=True, padding_mode="reflection").squeeze(0)


class TrivialAugmentWide:
    """One random op of random magnitude per sample."""

    def __init__(self):
        self.ops = [lambda x, m: x, lambda x, m: ColorJitter(brightness=m)(x), lambda x, m: ColorJitter(contrast=m)(x),
                    lambda x, m: RandomRotation(135 * m)(x), lambda x, m: GaussianNoise(0.2 * m)(x),
                    lambda x, m: (x > m).to(x) * x + (x <= m).to(x) * (1 - x)]

    def __call__(self, x):
        i = _vision_rng.randint(len(self.ops))
        return self.ops[i](x, _vision_rng.random())
