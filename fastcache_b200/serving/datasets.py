"""Workload loaders of the serving harness: LLaVA instruction mix (GQA subset), MileBench image
folders, and a synthetic generator for machines without the datasets.

Parity: scripts/llava_testcon2.6.py:1803-1925 (`load_image_data`, `load_image_data_milebench`) and the
two-sample demo file datasets/llava_v1_5_mix665k_demo.json.  Every loader returns a list of
`Sample(prompt, image, answers)`; `image` is a PIL image when the file exists and Pillow is
installed, a path string when it is only named, or a tensor for synthetic samples.  The prompt is
the reference's fixed description request, with `<image>` where the image rows go.
"""
from __future__ import annotations

import json
import random
from dataclasses import dataclass, field
from pathlib import Path
from typing import Any, List, Optional, Sequence

DESCRIBE_PROMPT = ("USER: <image> \nWhat's the content of the image? I am sick. Please describe every detail in the "
                   "image with specific and detailed language. ASSISTANT:")
IMAGE_SUFFIXES = (".jpg", ".jpeg", ".png", ".gif", ".bmp", ".tiff")


@dataclass
class Sample:
    prompt: str
    image: Any = None
    answers: List[str] = field(default_factory=list)
    source: str = ""


def _open_image(path: Path, must_exist: bool) -> Any:
    if not path.exists():
        if must_exist:
            raise FileNotFoundError(path)
        return str(path)
    try:
        from PIL import Image
    except ImportError:
        return str(path)
    try:
        return Image.open(path).convert("RGB")
    except Exception:                     # unreadable file: the caller still gets the path to report
        if must_exist:
            raise
        return str(path)


def load_image_data(json_path: str, imgsets_path: str, num_samples: int = -1,
                    target_datasets: Sequence[str] = ("gqa",), seed: Optional[int] = None,
                    must_exist: bool = False) -> List[Sample]:
    """Entries of a `llava_v1_5_mix665k`-style JSON whose image lives under one of `target_datasets`
    (first path component), shuffled, the first `num_samples` of them (< 0: all).  A conversation that
    opens with the human turn yields one sample; the assistant turns are kept as reference answers."""
    with open(json_path, "r", encoding="utf-8") as fh:
        data = json.load(fh)
    rows = [d for d in data if "image" in d and str(d["image"]).split("/")[0] in target_datasets]
    random.Random(seed).shuffle(rows)
    if num_samples >= 0:
        rows = rows[:num_samples]
    out: List[Sample] = []
    for d in rows:
        conv = d.get("conversations") or []
        if not conv or conv[0].get("from") != "human":
            continue
        answers = [t["value"] for t in conv if t.get("from") != "human"]
        out.append(Sample(DESCRIBE_PROMPT, _open_image(Path(imgsets_path) / d["image"], must_exist), answers,
                          source=str(d.get("id", d["image"]))))
    return out


def load_image_data_milebench(imgsets_path: str, num_samples: int = -1, seed: Optional[int] = None) -> List[Sample]:
    """MileBench layout: every folder `<name>/` that holds `<name>.json` and an `images/` sub-folder
    contributes all image files below `images/` (recursively, sorted); the union is shuffled."""
    root = Path(imgsets_path)
    paths: List[Path] = []
    for folder in sorted(p for p in root.rglob("*") if p.is_dir()):
        if not (folder / f"{folder.name}.json").exists() or not (folder / "images").is_dir():
            continue
        paths.extend(sorted(p for p in (folder / "images").rglob("*")
                            if p.is_file() and p.suffix.lower() in IMAGE_SUFFIXES))
    random.Random(seed).shuffle(paths)
    if num_samples >= 0:
        paths = paths[:num_samples]
    return [Sample(DESCRIBE_PROMPT, _open_image(p, False), [], source=str(p)) for p in paths]


def synthetic_samples(num_samples: int, image_hw=(336, 336), text_tokens: int = 64, vocab: int = 32000,
                      seed: int = 0) -> List[Sample]:
    """Uniform-random images in [0, 1] and uniform-random token-id prompts (lists of ints)."""
    import torch
    g = torch.Generator().manual_seed(seed)
    out = []
    for i in range(num_samples):
        ids = torch.randint(1000, max(1001, vocab - 1000), (text_tokens,), generator=g).tolist()
        out.append(Sample(ids, torch.rand(3, image_hw[0], image_hw[1], generator=g), [], source=f"synthetic-{i}"))
    return out
