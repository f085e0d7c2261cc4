"""Image-folder dataset for the ViT demos (reference: lib/core/data/image_folder_dataset.dart:1-287).

``root/<class name>/*.{jpg,jpeg,png}``: classes are the sorted sub-directories that hold at least one image, files are
sorted, capped at ``max_per_class``, shuffled with the split RNG and the first ``round(cap * val_split)`` go to the
validation split.  Images are decoded, resized bilinearly to ``image_size`` squared, scaled to ``[0, 1]`` RGB and
served pre-patchified: ``[numPatches, P*P*3]`` rows in ``(dy, dx, c)`` order, patches row-major.  ``val_split()`` shares
the decoded pixels; ``sample_triplet()`` draws (anchor, positive, negative) for metric learning.
"""
from __future__ import annotations

import os
import random
from dataclasses import dataclass
from typing import List, Optional

import numpy as np
import torch

from .datasets import Dataset


@dataclass
class FaceSample:
    patches: torch.Tensor
    label: int


@dataclass
class TripletSample:
    anchor: torch.Tensor
    positive: torch.Tensor
    negative: torch.Tensor
    anchor_class: int
    negative_class: int


_EXTS = (".jpg", ".jpeg", ".png")


class ImageFolderDataset(Dataset):
    def __init__(self, root_path: str, image_size: int, patch_size: int, max_per_class: int = 1 << 30,
                 max_classes: Optional[int] = None, val_split: float = 0.2, device=None, seed: int = 7,
                 val: bool = False, _shared: Optional["ImageFolderDataset"] = None):
        self.root_path, self.image_size, self.patch_size = root_path, image_size, patch_size
        self.device = device
        self._is_val = val
        if _shared is not None:
            self.classes, self._train, self._val = _shared.classes, _shared._train, _shared._val
            self._train_by_class, self._rng = _shared._train_by_class, _shared._rng
            return
        if image_size % patch_size:
            raise ValueError(f"imageSize ({image_size}) must be divisible by patchSize ({patch_size})")
        if not os.path.isdir(root_path):
            raise ValueError(f"rootPath does not exist: {root_path}")
        self._rng = random.Random(seed)
        split_rng = random.Random(seed)
        self.classes: List[str] = []
        self._train: List[tuple] = []
        self._val: List[tuple] = []
        class_dirs = sorted(e.path for e in os.scandir(root_path) if e.is_dir())
        if max_classes is not None:
            class_dirs = class_dirs[:max_classes]
        for cdir in class_dirs:
            files = sorted(e.path for e in os.scandir(cdir) if e.is_file() and e.name.lower().endswith(_EXTS))
            if not files:
                continue
            cap = min(len(files), max_per_class)
            self.classes.append(os.path.basename(cdir))
            label = len(self.classes) - 1
            order = list(range(cap))
            split_rng.shuffle(order)
            n_val = int(round(cap * val_split))
            for k, idx in enumerate(order):
                flat = self._decode(files[idx])
                if flat is None:
                    continue
                (self._val if k < n_val else self._train).append((flat, label))
        self._train_by_class: List[List[int]] = [[] for _ in self.classes]
        for i, (_, label) in enumerate(self._train):
            self._train_by_class[label].append(i)

    # ---- sizes ------------------------------------------------------------------------------------
    @property
    def num_classes(self) -> int:
        return len(self.classes)

    @property
    def num_train(self) -> int:
        return len(self._train)

    @property
    def num_val(self) -> int:
        return len(self._val)

    @property
    def patch_pixels(self) -> int:
        return self.patch_size * self.patch_size * 3

    @property
    def num_patches(self) -> int:
        return (self.image_size // self.patch_size) ** 2

    numClasses, numTrain, numVal, patchPixels, numPatches = num_classes, num_train, num_val, patch_pixels, num_patches

    # ---- decoding ---------------------------------------------------------------------------------
    def _decode(self, path: str) -> Optional[np.ndarray]:
        """``[H, W, 3]`` float32 in ``[0, 1]``, or ``None`` for an unreadable file (skipped, as in the reference)."""
        try:
            from PIL import Image
            with Image.open(path) as im:
                im = im.convert("RGB").resize((self.image_size, self.image_size), Image.BILINEAR)
                return np.asarray(im, dtype=np.float32) / 255.0
        except Exception:
            return None

    def patchify(self, flat: np.ndarray) -> np.ndarray:
        """``[H, W, 3]`` (or the same flattened) -> ``[numPatches, P*P*3]``."""
        s, p = self.image_size, self.patch_size
        g = s // p
        img = np.asarray(flat, dtype=np.float32).reshape(s, s, 3)
        return img.reshape(g, p, g, p, 3).transpose(0, 2, 1, 3, 4).reshape(g * g, p * p * 3)

    def _as_tensor(self, flat: np.ndarray) -> torch.Tensor:
        t = torch.from_numpy(np.ascontiguousarray(self.patchify(flat)))
        return t.to(self.device) if self.device is not None else t

    # ---- dataset protocol -------------------------------------------------------------------------
    def __len__(self) -> int:
        return len(self._val) if self._is_val else len(self._train)

    def __getitem__(self, index: int) -> FaceSample:
        flat, label = (self._val if self._is_val else self._train)[index]
        return FaceSample(self._as_tensor(flat), label)

    def val_split(self) -> "ImageFolderDataset":
        if self._is_val:
            return self
        return ImageFolderDataset(self.root_path, self.image_size, self.patch_size, device=self.device, val=True,
                                  _shared=self)

    valSplit = val_split

    # ---- triplets ---------------------------------------------------------------------------------
    @property
    def triplet_ready_classes(self) -> List[int]:
        return [c for c, idx in enumerate(self._train_by_class) if len(idx) >= 2]

    tripletReadyClasses = triplet_ready_classes

    def sample_triplet(self) -> TripletSample:
        ready = self.triplet_ready_classes
        if len(ready) < 2:
            raise RuntimeError(f"Need >= 2 classes with >= 2 train samples each for triplets, got {len(ready)}")
        a_class = ready[self._rng.randrange(len(ready))]
        n_class = a_class
        while n_class == a_class:
            n_class = ready[self._rng.randrange(len(ready))]
        a_list = self._train_by_class[a_class]
        i1 = self._rng.randrange(len(a_list))
        i2 = i1
        while i2 == i1:
            i2 = self._rng.randrange(len(a_list))
        n_list = self._train_by_class[n_class]
        i3 = self._rng.randrange(len(n_list))
        return TripletSample(self._as_tensor(self._train[a_list[i1]][0]), self._as_tensor(self._train[a_list[i2]][0]),
                             self._as_tensor(self._train[n_list[i3]][0]), a_class, n_class)

    sampleTriplet = sample_triplet
