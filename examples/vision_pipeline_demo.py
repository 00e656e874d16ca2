"""Image transforms, preprocessing pipelines with caching and statistics, presets, and a dataset written and read in
the MNIST file format."""
import _path  # noqa: F401
import os
import tempfile

import numpy as np
import torch

from rustorch_b200 import vision as V

torch.manual_seed(0)
img = torch.rand(3, 48, 64)
aug = V.Compose([V.Resize((40, 40)), V.RandomCrop(32, padding=2), V.RandomHorizontalFlip(0.5), V.ColorJitter(0.2, 0.2, 0.2),
                 V.Normalize(V.IMAGENET_MEAN, V.IMAGENET_STD)])
print("augmented:", tuple(aug(img).shape), " centre crop:", tuple(V.CenterCrop(24)(img).shape))
pipe = (V.PipelineBuilder("eval").transform(V.Resize(36)).conditional(V.CenterCrop(32), lambda t: t.shape[-1] > 32)
        .transform(V.Normalize([0.5] * 3, [0.5] * 3)).cache(8).build())
for key in ("a", "b", "a", "a"):
    out = pipe(img, key=key)
print("pipeline output", tuple(out.shape), "processed", pipe.stats.total_processed, "cache hits", pipe.stats.cache_hits,
      "stages", list(pipe.stats.per_transform_s))
print("ImageNet validation preset:", tuple(V.ImageNetPreprocessing.validation()(torch.rand(3, 300, 280) * 255).shape),
      " CIFAR training preset:", tuple(V.CIFARPreprocessing.training()(torch.rand(3, 32, 32)).shape))
root = tempfile.mkdtemp()
V.write_idx(os.path.join(root, "train-images-idx3-ubyte.gz"), (np.random.rand(16, 28, 28) * 255).astype(np.uint8))
V.write_idx(os.path.join(root, "train-labels-idx1-ubyte"), (np.arange(16) % 10).astype(np.uint8))
ds = V.MNIST(root, train=True)
x0, y0 = ds[3]
print("MNIST files:", len(ds), "samples; sample 3:", tuple(x0.shape), "label", int(y0))
grid = V.make_grid(torch.stack([ds[i][0] for i in range(8)]), nrow=4)
V.save_image(grid, os.path.join(root, "grid.pgm"))
print("grid", tuple(grid.shape), "written:", os.path.getsize(os.path.join(root, "grid.pgm")), "bytes")
