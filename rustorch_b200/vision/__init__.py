"""Vision: ``Image`` container, transforms, pipelines, presets and dataset readers
(src/vision/mod.rs:26-60, transforms.rs:18-420, pipeline.rs:21-450, presets.rs:18-230, datasets.rs:22-700).

Transforms operate on ``[C, H, W]`` or batched ``[N, C, H, W]`` tensors on whatever device they live on, so a
batch can be augmented on the GPU after one pinned-memory copy instead of per image on the host (the
reference transforms one image at a time on the CPU).  Dataset classes read the standard on-disk formats
(MNIST IDX, CIFAR binary batches, image folders of ``.npy`` / ``.ppm`` / ``.pgm`` files); nothing is downloaded.
"""
from __future__ import annotations

import gzip
import math
import os
import struct
import time
from dataclasses import dataclass, field
from enum import Enum
from typing import Callable, Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch
import torch.nn.functional as F


class ImageFormat(Enum):
    """Channel layout of an image tensor: CHW or HWC (src/vision/mod.rs)."""

    CHW = "chw"
    HWC = "hwc"


@dataclass
class Image:
    """A tensor plus its layout; ``to_chw`` / ``to_hwc`` convert."""
    data: torch.Tensor
    format: ImageFormat = ImageFormat.CHW

    @property
    def height(self) -> int:
        return self.data.shape[1 if self.format is ImageFormat.CHW else 0]

    @property
    def width(self) -> int:
        return self.data.shape[2 if self.format is ImageFormat.CHW else 1]

    @property
    def channels(self) -> int:
        return self.data.shape[0 if self.format is ImageFormat.CHW else 2]

    def to_chw(self) -> "Image":
        return self if self.format is ImageFormat.CHW else Image(self.data.permute(2, 0, 1).contiguous(), ImageFormat.CHW)

    def to_hwc(self) -> "Image":
        return self if self.format is ImageFormat.HWC else Image(self.data.permute(1, 2, 0).contiguous(), ImageFormat.HWC)


def _t(x) -> torch.Tensor:
    return x.to_chw().data if isinstance(x, Image) else x


class Transform:
    def __call__(self, x):
        return self.apply(_t(x))

    def apply(self, x: torch.Tensor) -> torch.Tensor:
        raise NotImplementedError

    @property
    def name(self) -> str:
        return type(self).__name__


class InterpolationMode(Enum):
    """Resampling filter of ``Resize``."""

    NEAREST = "nearest"
    BILINEAR = "bilinear"
    BICUBIC = "bicubic"


class Resize(Transform):
    def __init__(self, size, interpolation: InterpolationMode = InterpolationMode.BILINEAR):
        self.size = (size, size) if isinstance(size, int) else tuple(size)
        self.interpolation = interpolation

    def apply(self, x):
        batched = x.dim() == 4
        xb = x if batched else x.unsqueeze(0)
        mode = self.interpolation.value
        kw = {} if mode == "nearest" else {"align_corners": False}
        y = F.interpolate(xb.float(), size=self.size, mode=mode, **kw).to(x.dtype if x.is_floating_point() else torch.float32)
        return y if batched else y[0]


class CenterCrop(Transform):
    def __init__(self, size):
        self.size = (size, size) if isinstance(size, int) else tuple(size)

    def apply(self, x):
        h, w = x.shape[-2:]
        th, tw = self.size
        if th > h or tw > w:
            raise ValueError(f"crop {self.size} larger than image {(h, w)}")
        i, j = (h - th) // 2, (w - tw) // 2
        return x[..., i:i + th, j:j + tw]


class RandomCrop(Transform):
    def __init__(self, size, padding: int = 0, generator: Optional[torch.Generator] = None):
        self.size = (size, size) if isinstance(size, int) else tuple(size)
        self.padding, self.generator = padding, generator

    def apply(self, x):
        if self.padding:
            x = F.pad(x, [self.padding] * 4)
        h, w = x.shape[-2:]
        th, tw = self.size
        if th > h or tw > w:
            raise ValueError(f"crop {self.size} larger than image {(h, w)}")
        i = int(torch.randint(0, h - th + 1, (1,), generator=self.generator))
        j = int(torch.randint(0, w - tw + 1, (1,), generator=self.generator))
        return x[..., i:i + th, j:j + tw]


class RandomHorizontalFlip(Transform):
    """Per-sample coin flip (vectorised over a batch)."""

    def __init__(self, p: float = 0.5, generator: Optional[torch.Generator] = None):
        self.p, self.generator = p, generator

    def apply(self, x):
        if x.dim() == 3:
            return x.flip(-1) if float(torch.rand(1, generator=self.generator)) < self.p else x
        flip = torch.rand(x.shape[0], generator=self.generator) < self.p
        return torch.where(flip.to(x.device).view(-1, 1, 1, 1), x.flip(-1), x)


class RandomVerticalFlip(RandomHorizontalFlip):
    def apply(self, x):
        if x.dim() == 3:
            return x.flip(-2) if float(torch.rand(1, generator=self.generator)) < self.p else x
        flip = torch.rand(x.shape[0], generator=self.generator) < self.p
        return torch.where(flip.to(x.device).view(-1, 1, 1, 1), x.flip(-2), x)


class RandomRotation(Transform):
    """Rotation by a random angle in ``[-degrees, degrees]`` about the centre (bilinear resampling)."""

    def __init__(self, degrees: float, generator: Optional[torch.Generator] = None):
        self.degrees, self.generator = float(degrees), generator

    def apply(self, x):
        batched = x.dim() == 4
        xb = (x if batched else x.unsqueeze(0)).float()
        n = xb.shape[0]
        ang = (torch.rand(n, generator=self.generator) * 2 - 1) * math.radians(self.degrees)
        cs, sn = torch.cos(ang), torch.sin(ang)
        theta = torch.stack([torch.stack([cs, -sn, torch.zeros(n)], 1), torch.stack([sn, cs, torch.zeros(n)], 1)], 1).to(xb.device)
        grid = F.affine_grid(theta, list(xb.shape), align_corners=False)
        y = F.grid_sample(xb, grid, mode="bilinear", padding_mode="zeros", align_corners=False)
        return y if batched else y[0]


class Normalize(Transform):
    def __init__(self, mean: Sequence[float], std: Sequence[float]):
        if any(s == 0 for s in std):
            raise ValueError("std must be non-zero")
        self.mean, self.std = torch.tensor(mean, dtype=torch.float32), torch.tensor(std, dtype=torch.float32)

    def apply(self, x):
        m = self.mean.to(x.device).view(-1, 1, 1)
        s = self.std.to(x.device).view(-1, 1, 1)
        return (x.float() - m) / s


class ToTensor(Transform):
    """uint8 HWC (numpy / tensor / ``Image``) -> float CHW in [0, 1]."""

    def __call__(self, x):
        if isinstance(x, Image):
            x = x.to_chw().data
        elif isinstance(x, np.ndarray):
            x = torch.from_numpy(x)
            x = x.permute(2, 0, 1) if x.dim() == 3 else x.unsqueeze(0)
        return self.apply(x)

    def apply(self, x):
        return x.float() / 255.0 if x.dtype == torch.uint8 else x.float()


class ColorJitter(Transform):
    """Random brightness, contrast, saturation and hue changes of ``[..., C, H, W]`` images in ``[0, 1]``; each factor is
    drawn uniformly from ``1 +- amount`` (hue: a rotation of the chroma plane by up to ``hue`` turns)."""

    def __init__(self, brightness: float = 0.0, contrast: float = 0.0, saturation: float = 0.0, hue: float = 0.0,
                 generator: Optional[torch.Generator] = None):
        if isinstance(saturation, torch.Generator):                   # (brightness, contrast, generator)
            saturation, generator = 0.0, saturation
        if min(brightness, contrast, saturation) < 0 or not 0.0 <= hue <= 0.5:
            raise ValueError("jitter amounts must be non-negative and hue at most 0.5")
        self.brightness, self.contrast, self.saturation, self.hue, self.generator = brightness, contrast, saturation, hue, generator

    def _draw(self, amount: float) -> float:
        return 1 + (float(torch.rand(1, generator=self.generator)) * 2 - 1) * amount

    def apply(self, x):
        x = x.float()
        b, c = self._draw(self.brightness), self._draw(self.contrast)
        mean = x.mean(dim=(-3, -2, -1), keepdim=True)
        x = ((x * b - mean) * c + mean).clamp(0, 1)
        if x.shape[-3] == 3 and (self.saturation or self.hue):
            wts = torch.tensor([0.299, 0.587, 0.114], device=x.device).view(3, 1, 1)
            grey = (x * wts).sum(-3, keepdim=True)
            if self.saturation:
                x = (grey + (x - grey) * self._draw(self.saturation)).clamp(0, 1)
            if self.hue:
                # rotate the chroma (I, Q) plane of YIQ by the drawn angle
                ang = (float(torch.rand(1, generator=self.generator)) * 2 - 1) * self.hue * 2 * math.pi
                to_yiq = torch.tensor([[0.299, 0.587, 0.114], [0.596, -0.274, -0.322], [0.211, -0.523, 0.312]], device=x.device)
                rot = torch.tensor([[1.0, 0.0, 0.0], [0.0, math.cos(ang), -math.sin(ang)], [0.0, math.sin(ang), math.cos(ang)]], device=x.device)
                m = torch.linalg.inv(to_yiq) @ rot @ to_yiq
                x = torch.einsum("ij,...jhw->...ihw", m, x).clamp(0, 1)
        return x


class Compose(Transform):
    """Applies transforms one after another (src/vision/transforms.rs)."""

    def __init__(self, transforms: Sequence[Callable]):
        self.transforms = list(transforms)

    def __call__(self, x):
        for t in self.transforms:
            x = t(x)
        return x


# ------------------------------------------------------------------------------ pipeline
class ExecutionMode(Enum):
    """Sequential, batched or parallel execution of a pipeline (src/vision/pipeline.rs)."""

    SEQUENTIAL = "sequential"
    BATCH = "batch"


@dataclass
class PipelineStats:
    total_processed: int = 0
    total_time_s: float = 0.0
    per_transform_s: Dict[str, float] = field(default_factory=dict)
    cache_hits: int = 0

    @property
    def images_per_s(self) -> float:
        return self.total_processed / self.total_time_s if self.total_time_s > 0 else 0.0


class ConditionalTransform(Transform):
    """Applies a transform only where a predicate on the image holds (src/vision/pipeline.rs)."""

    def __init__(self, transform: Callable, predicate: Callable[[torch.Tensor], bool]):
        self.transform, self.predicate = transform, predicate

    def __call__(self, x):
        return self.transform(x) if self.predicate(_t(x)) else _t(x)


class Pipeline:
    """Named chain of transforms with timing statistics and an optional keyed result cache."""

    def __init__(self, name: str = "pipeline", mode: ExecutionMode = ExecutionMode.SEQUENTIAL, cache_size: int = 0):
        self.name, self.mode = name, mode
        self.transforms: List[Tuple[str, Callable]] = []
        self.stats = PipelineStats()
        self._cache: Dict[object, torch.Tensor] = {}
        self.cache_size = cache_size

    def add(self, transform: Callable, name: Optional[str] = None) -> "Pipeline":
        self.transforms.append((name or getattr(transform, "name", type(transform).__name__), transform))
        return self

    def __call__(self, x, key=None):
        if key is not None and key in self._cache:
            self.stats.cache_hits += 1
            return self._cache[key]
        t0 = time.perf_counter()
        for n, t in self.transforms:
            s = time.perf_counter()
            x = t(x)
            self.stats.per_transform_s[n] = self.stats.per_transform_s.get(n, 0.0) + time.perf_counter() - s
        self.stats.total_time_s += time.perf_counter() - t0
        self.stats.total_processed += x.shape[0] if isinstance(x, torch.Tensor) and x.dim() == 4 else 1
        if key is not None and self.cache_size:
            if len(self._cache) >= self.cache_size:
                self._cache.pop(next(iter(self._cache)))
            self._cache[key] = x
        return x

    def process_batch(self, images: Sequence) -> List[torch.Tensor]:
        if self.mode is ExecutionMode.BATCH and all(isinstance(i, torch.Tensor) and i.shape == images[0].shape for i in images):
            return list(self(torch.stack(list(images))))
        return [self(i) for i in images]


class PipelineBuilder:
    def __init__(self, name: str = "pipeline"):
        self._p = Pipeline(name)

    def transform(self, t: Callable, name: Optional[str] = None) -> "PipelineBuilder":
        self._p.add(t, name)
        return self

    def conditional(self, t: Callable, predicate) -> "PipelineBuilder":
        self._p.add(ConditionalTransform(t, predicate), f"if:{getattr(t, 'name', 'transform')}")
        return self

    def execution_mode(self, mode: ExecutionMode) -> "PipelineBuilder":
        self._p.mode = mode
        return self

    def cache(self, size: int) -> "PipelineBuilder":
        self._p.cache_size = size
        return self

    def build(self) -> Pipeline:
        return self._p


# ------------------------------------------------------------------------------ presets
IMAGENET_MEAN, IMAGENET_STD = (0.485, 0.456, 0.406), (0.229, 0.224, 0.225)
CIFAR_MEAN, CIFAR_STD = (0.4914, 0.4822, 0.4465), (0.2470, 0.2435, 0.2616)


class ImageNetPreprocessing:
    @staticmethod
    def training() -> Pipeline:
        return (PipelineBuilder("imagenet_train").transform(Resize(256)).transform(RandomCrop(224))
                .transform(RandomHorizontalFlip()).transform(ToTensor()).transform(Normalize(IMAGENET_MEAN, IMAGENET_STD)).build())

    @staticmethod
    def validation() -> Pipeline:
        return (PipelineBuilder("imagenet_val").transform(Resize(256)).transform(CenterCrop(224)).transform(ToTensor())
                .transform(Normalize(IMAGENET_MEAN, IMAGENET_STD)).build())


class CIFARPreprocessing:
    @staticmethod
    def training() -> Pipeline:
        return (PipelineBuilder("cifar_train").transform(RandomCrop(32, padding=4)).transform(RandomHorizontalFlip())
                .transform(ToTensor()).transform(Normalize(CIFAR_MEAN, CIFAR_STD)).build())

    @staticmethod
    def validation() -> Pipeline:
        return PipelineBuilder("cifar_val").transform(ToTensor()).transform(Normalize(CIFAR_MEAN, CIFAR_STD)).build()


class ObjectDetectionPreprocessing:
    @staticmethod
    def pipeline(size: int = 416) -> Pipeline:
        return PipelineBuilder("detection").transform(Resize(size)).transform(ToTensor()).build()


class SegmentationPreprocessing:
    @staticmethod
    def pipeline(size: int = 512) -> Pipeline:
        return (PipelineBuilder("segmentation").transform(Resize(size, InterpolationMode.NEAREST)).transform(ToTensor()).build())


class MedicalImagingPreprocessing:
    @staticmethod
    def pipeline(size: int = 512) -> Pipeline:
        return (PipelineBuilder("medical").transform(Resize(size)).transform(CenterCrop(size)).transform(ToTensor())
                .transform(Normalize((0.5,), (0.5,))).build())


class MobileOptimizedPreprocessing:
    @staticmethod
    def pipeline(size: int = 160) -> Pipeline:
        return (PipelineBuilder("mobile").transform(Resize(size, InterpolationMode.NEAREST)).transform(ToTensor())
                .transform(Normalize(IMAGENET_MEAN, IMAGENET_STD)).build())


class CustomPipelineFactory:
    @staticmethod
    def create(size: int, mean: Sequence[float], std: Sequence[float], augment: bool = False) -> Pipeline:
        b = PipelineBuilder("custom").transform(Resize(size))
        if augment:
            b.transform(RandomHorizontalFlip())
        return b.transform(ToTensor()).transform(Normalize(mean, std)).build()


# ------------------------------------------------------------------------------ datasets
def _open(path: str):
    return gzip.open(path, "rb") if path.endswith(".gz") else open(path, "rb")


def read_idx(path: str) -> np.ndarray:
    """IDX file (MNIST): magic ``00 00 dtype ndim`` · big-endian dims · data."""
    with _open(path) as f:
        zero, dtype, ndim = struct.unpack(">HBB", f.read(4))
        if zero != 0:
            raise ValueError(f"{path}: bad IDX magic")
        dims = struct.unpack(f">{ndim}I", f.read(4 * ndim))
        dt = {0x08: np.uint8, 0x09: np.int8, 0x0B: ">i2", 0x0C: ">i4", 0x0D: ">f4", 0x0E: ">f8"}[dtype]
        return np.frombuffer(f.read(), dtype=dt).reshape(dims)


def write_idx(path: str, arr: np.ndarray) -> None:
    code = {np.dtype(np.uint8): 0x08, np.dtype(np.int8): 0x09}[arr.dtype]
    with (gzip.open(path, "wb") if path.endswith(".gz") else open(path, "wb")) as f:
        f.write(struct.pack(">HBB", 0, code, arr.ndim) + struct.pack(f">{arr.ndim}I", *arr.shape) + arr.tobytes())


class _ArrayDataset:
    classes: List[str] = []

    def __init__(self, images: np.ndarray, labels: np.ndarray, transform: Optional[Callable] = None):
        self.images, self.labels, self.transform = images, labels.astype(np.int64), transform

    def __len__(self) -> int:
        return len(self.labels)

    def __getitem__(self, i: int):
        img = torch.from_numpy(np.ascontiguousarray(self.images[i]))
        img = self.transform(img) if self.transform else img.float() / 255.0
        return img, int(self.labels[i])

    def as_tensors(self) -> Tuple[torch.Tensor, torch.Tensor]:
        """Whole split as ``(uint8 [N, C, H, W], int64 [N])``: one pinned copy to the GPU, augment there."""
        return torch.from_numpy(np.ascontiguousarray(self.images)), torch.from_numpy(self.labels)


class MNIST(_ArrayDataset):
    """MNIST from the IDX files, gzip or plain (src/vision/datasets.rs)."""

    classes = [str(i) for i in range(10)]

    def __init__(self, root: str, train: bool = True, transform: Optional[Callable] = None):
        stem = "train" if train else "t10k"
        def find(kind):
            for suffix in ("", ".gz"):
                for sep in ("-", "."):
                    p = os.path.join(root, f"{stem}-{kind}{sep}idx{'3' if kind == 'images' else '1'}-ubyte{suffix}")
                    if os.path.exists(p):
                        return p
            raise FileNotFoundError(f"MNIST {stem} {kind} file not found under {root} (nothing is downloaded)")
        imgs = read_idx(find("images"))
        super().__init__(imgs[:, None, :, :], read_idx(find("labels")), transform)


class CIFAR10(_ArrayDataset):
    """CIFAR-10 from the binary batch files (src/vision/datasets.rs)."""

    classes = ["airplane", "automobile", "bird", "cat", "deer", "dog", "frog", "horse", "ship", "truck"]
    _label_bytes, _label_index = 1, 0

    def __init__(self, root: str, train: bool = True, transform: Optional[Callable] = None):
        files = self._files(train)
        rec = self._label_bytes + 3072
        imgs, labels = [], []
        for fn in files:
            p = os.path.join(root, fn)
            if not os.path.exists(p):
                raise FileNotFoundError(f"{p} not found (nothing is downloaded)")
            raw = np.fromfile(p, dtype=np.uint8)
            if raw.size % rec:
                raise ValueError(f"{p}: size is not a multiple of the {rec}-byte record")
            raw = raw.reshape(-1, rec)
            labels.append(raw[:, self._label_index])
            imgs.append(raw[:, self._label_bytes:].reshape(-1, 3, 32, 32))
        super().__init__(np.concatenate(imgs), np.concatenate(labels), transform)

    def _files(self, train: bool) -> List[str]:
        return [f"data_batch_{i}.bin" for i in range(1, 6)] if train else ["test_batch.bin"]


class CIFAR100(CIFAR10):
    """Binary records are ``coarse label · fine label · 3072 pixels``; fine labels are returned."""
    classes = [str(i) for i in range(100)]
    _label_bytes, _label_index = 2, 1

    def _files(self, train: bool) -> List[str]:
        return ["train.bin"] if train else ["test.bin"]


def read_pnm(path: str) -> np.ndarray:
    """Binary PGM (P5) / PPM (P6), 8-bit -> HWC uint8."""
    with open(path, "rb") as f:
        data = f.read()
    tokens, i = [], 0
    while len(tokens) < 4:
        while data[i:i + 1].isspace():
            i += 1
        if data[i:i + 1] == b"#":
            while data[i:i + 1] != b"\n":
                i += 1
            continue
        j = i
        while not data[j:j + 1].isspace():
            j += 1
        tokens.append(data[i:j])
        i = j
    magic, w, h, mx = tokens[0], int(tokens[1]), int(tokens[2]), int(tokens[3])
    if magic not in (b"P5", b"P6") or mx > 255:
        raise ValueError(f"{path}: only 8-bit binary PGM/PPM supported")
    c = 1 if magic == b"P5" else 3
    return np.frombuffer(data, dtype=np.uint8, count=w * h * c, offset=i + 1).reshape(h, w, c)


class ImageFolder:
    """``root/<class>/<file>`` with ``.npy`` (HWC or CHW uint8/float), ``.ppm`` or ``.pgm`` files."""

    EXT = (".npy", ".ppm", ".pgm")

    def __init__(self, root: str, transform: Optional[Callable] = None):
        self.classes = sorted(d for d in os.listdir(root) if os.path.isdir(os.path.join(root, d)))
        if not self.classes:
            raise FileNotFoundError(f"no class folders under {root}")
        self.class_to_idx = {c: i for i, c in enumerate(self.classes)}
        self.samples = [(os.path.join(root, c, f), self.class_to_idx[c]) for c in self.classes
                        for f in sorted(os.listdir(os.path.join(root, c))) if f.lower().endswith(self.EXT)]
        self.transform = transform

    def __len__(self) -> int:
        return len(self.samples)

    def __getitem__(self, i: int):
        path, label = self.samples[i]
        arr = np.load(path) if path.endswith(".npy") else read_pnm(path)
        t = torch.from_numpy(np.ascontiguousarray(arr))
        if t.dim() == 3 and t.shape[-1] in (1, 3, 4) and t.shape[0] not in (1, 3, 4):
            t = t.permute(2, 0, 1)
        elif t.dim() == 2:
            t = t.unsqueeze(0)
        t = self.transform(t) if self.transform else (t.float() / 255.0 if t.dtype == torch.uint8 else t.float())
        return t, label


def make_grid(images, nrow: int = 8, padding: int = 2, pad_value: float = 0.0) -> torch.Tensor:
    """``[N, C, H, W]`` (or a list of ``[C, H, W]``) tiled into one ``[C, rows * (H + p) + p, cols * (W + p) + p]`` image
    (src/vision/utils.rs make_grid)."""
    x = torch.stack([_t(i) for i in images]) if not isinstance(images, torch.Tensor) else images
    if x.dim() == 3:
        x = x.unsqueeze(0)
    n, c, h, w = x.shape
    cols = min(nrow, n)
    rows = -(-n // cols)
    grid = torch.full((c, rows * (h + padding) + padding, cols * (w + padding) + padding), pad_value, dtype=x.dtype)
    for i in range(n):
        r, q = divmod(i, cols)
        top, left = padding + r * (h + padding), padding + q * (w + padding)
        grid[:, top:top + h, left:left + w] = x[i]
    return grid


def save_image(image, path: str, nrow: int = 8, padding: int = 2) -> None:
    """Writes a ``[C, H, W]`` image (or a batch, tiled with ``make_grid``) with values in [0, 1] as PNG."""
    from ..tensorboard import encode_png
    x = image if isinstance(image, torch.Tensor) else torch.stack([_t(i) for i in image])
    if x.dim() == 4:
        x = make_grid(x, nrow, padding)
    arr = (x.detach().float().clamp(0, 1) * 255).round().to(torch.uint8).permute(1, 2, 0).cpu().numpy()
    with open(path, "wb") as f:
        f.write(encode_png(arr))
