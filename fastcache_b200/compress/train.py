"""Training of the CCM merge compressors by distillation.

Parity:
  * KVCacheCompressionLoss   utils_ccm/module_ccm_v11.py:1281-1867 — cross-entropy on labels plus
    Jensen-Shannon and L1 terms between the output distributions obtained with the compressed and the
    original KV, and per-layer hidden-state MSE + cosine terms; strategies logit / label /
    label_twice / label_confident.
  * fine-tune loops          scripts/finetune_llava.py:509-791, scripts/finetune_minicpm.py:863-1195 —
    Adam(lr 5e-4), ReduceLROnPlateau, ratio 5, "original twice" teacher forward, `last_` / `best_`
    checkpoints in the layout of `save_compressor`, resume with `is_continue`.
The loop here is model-agnostic: the caller supplies `forward_with_kv(batch, kv or None) ->
(logits, hidden_states, kv)` so it runs with a HuggingFace model or with a toy model in tests.
"""
from __future__ import annotations

import os
from dataclasses import dataclass
from typing import Any, Callable, Dict, Iterable, List, Optional, Sequence, Tuple

import torch
import torch.nn.functional as F
from torch import nn

from .ccm import _CCMBase, save_compressor


class KVCacheCompressionLoss(nn.Module):
    def __init__(self, strategy: str = "logit", ce_weight: float = 1.0, js_weight: float = 1.0,
                 l1_weight: float = 0.1, hidden_mse_weight: float = 0.1, hidden_cos_weight: float = 0.1,
                 temperature: float = 1.0, confident_top_p: float = 0.9):
        super().__init__()
        if strategy not in ("logit", "label", "label_twice", "label_confident"):
            raise ValueError(strategy)
        self.strategy = strategy
        self.w = dict(ce=ce_weight, js=js_weight, l1=l1_weight, mse=hidden_mse_weight, cos=hidden_cos_weight)
        self.temperature = temperature
        self.confident_top_p = confident_top_p

    @staticmethod
    def js_divergence(p_logits: torch.Tensor, q_logits: torch.Tensor) -> torch.Tensor:
        p, q = F.softmax(p_logits.float(), -1), F.softmax(q_logits.float(), -1)
        m = 0.5 * (p + q)
        kl = lambda a, b: (a * (a.clamp_min(1e-12).log() - b.clamp_min(1e-12).log())).sum(-1)  # noqa: E731
        return 0.5 * (kl(p, m) + kl(q, m)).mean()

    def forward(self, student_logits: torch.Tensor, teacher_logits: torch.Tensor,
                labels: Optional[torch.Tensor] = None,
                student_hidden: Optional[Sequence[torch.Tensor]] = None,
                teacher_hidden: Optional[Sequence[torch.Tensor]] = None) -> Tuple[torch.Tensor, Dict[str, float]]:
        t = self.temperature
        parts: Dict[str, torch.Tensor] = {}
        V = student_logits.shape[-1]
        s2, t2 = student_logits.reshape(-1, V), teacher_logits.reshape(-1, V).detach()
        if self.strategy == "logit":
            parts["js"] = self.js_divergence(s2 / t, t2 / t)
            parts["l1"] = (F.softmax(s2.float(), -1) - F.softmax(t2.float(), -1)).abs().sum(-1).mean()
        if self.strategy in ("label", "label_twice") and labels is not None:
            parts["ce"] = F.cross_entropy(s2.float(), labels.reshape(-1), ignore_index=-100)
        if self.strategy in ("label_twice", "label_confident", "logit"):
            pseudo = t2.argmax(-1)
            if self.strategy == "label_confident":
                conf = F.softmax(t2.float(), -1).max(-1).values
                pseudo = torch.where(conf >= self.confident_top_p, pseudo, torch.full_like(pseudo, -100))
            if (pseudo != -100).any():
                key = "ce_teacher" if "ce" in parts else "ce"
                parts[key] = F.cross_entropy(s2.float(), pseudo, ignore_index=-100)
        if student_hidden is not None and teacher_hidden is not None:
            mse = cos = 0.0
            n = min(len(student_hidden), len(teacher_hidden))
            for a, b in zip(student_hidden[:n], teacher_hidden[:n]):
                mse = mse + F.mse_loss(a.float(), b.detach().float())
                cos = cos + (1.0 - F.cosine_similarity(a.float(), b.detach().float(), dim=-1).mean())
            parts["mse"], parts["cos"] = mse / max(1, n), cos / max(1, n)
        total = sum(self.w.get(k.split("_")[0], 1.0) * v for k, v in parts.items())
        return total, {k: float(v.detach()) if torch.is_tensor(v) else float(v) for k, v in parts.items()}

    @staticmethod
    def accuracy(student_logits: torch.Tensor, teacher_logits: torch.Tensor) -> float:
        """Share of positions where the compressed-KV prediction equals the original-KV prediction."""
        return float((student_logits.argmax(-1) == teacher_logits.argmax(-1)).float().mean())


@dataclass
class FinetuneConfig:
    lr: float = 5e-4
    epochs: int = 40
    compression_factor: int = 5
    out_dir: str = "ckpt"
    name: str = "compressor"
    is_continue: bool = False
    plateau_patience: int = 2
    plateau_factor: float = 0.5
    grad_clip: float = 1.0


def finetune_compressor(compressor: _CCMBase,
                        forward_with_kv: Callable[[Any, Optional[List[Tuple[torch.Tensor, torch.Tensor]]]],
                                                  Tuple[torch.Tensor, Sequence[torch.Tensor],
                                                        List[Tuple[torch.Tensor, torch.Tensor]]]],
                        train_batches: Iterable[Any], val_batches: Iterable[Any], cfg: FinetuneConfig,
                        it_len_of: Callable[[Any], Sequence[int]] = lambda b: (0, 0),
                        loss_fn: Optional[KVCacheCompressionLoss] = None) -> Dict[str, Any]:
    """Distil the compressor: the teacher is the model run on the original KV, the student the same
    model run on the compressed KV.  `forward_with_kv(batch, None)` runs the prefix and returns its KV;
    `forward_with_kv(batch, kv)` runs the continuation on the given KV."""
    loss_fn = loss_fn or KVCacheCompressionLoss("logit")
    compressor.train()
    opt = torch.optim.Adam(compressor.parameters(), lr=cfg.lr)
    sched = torch.optim.lr_scheduler.ReduceLROnPlateau(opt, factor=cfg.plateau_factor, patience=cfg.plateau_patience)
    os.makedirs(cfg.out_dir, exist_ok=True)
    last = os.path.join(cfg.out_dir, f"last_{cfg.name}.pth")
    best = os.path.join(cfg.out_dir, f"best_{cfg.name}.pth")
    start, best_val = 0, float("inf")
    if cfg.is_continue and os.path.exists(last):
        blob = torch.load(last, map_location="cpu", weights_only=False)
        compressor.load_state_dict(blob["model_state_dict"]["compressor"])
        if blob.get("optimizer_state_dict"):
            opt.load_state_dict(blob["optimizer_state_dict"])
        if blob.get("scheduler_state_dict"):
            sched.load_state_dict(blob["scheduler_state_dict"])
        start, best_val = int(blob.get("epoch", 0)) + 1, float(blob.get("loss", best_val))
    history: List[Dict[str, float]] = []

    def run(batch: Any, train: bool) -> Tuple[torch.Tensor, float]:
        with torch.no_grad():
            _, _, kv = forward_with_kv(batch, None)
            t_logits, t_hidden, _ = forward_with_kv(batch, kv)                 # "original twice" teacher
        ckv = _compress_with_grad(compressor, kv, it_len_of(batch)) if train else compressor(kv, it_len_of(batch))
        s_logits, s_hidden, _ = forward_with_kv(batch, ckv)
        loss, _ = loss_fn(s_logits, t_logits, None, s_hidden, t_hidden)
        return loss, loss_fn.accuracy(s_logits, t_logits)

    for epoch in range(start, cfg.epochs):
        compressor.train()
        tot = n = 0.0
        for batch in train_batches:
            opt.zero_grad(set_to_none=True)
            loss, _ = run(batch, True)
            loss.backward()
            if cfg.grad_clip:
                nn.utils.clip_grad_norm_(compressor.parameters(), cfg.grad_clip)
            opt.step()
            tot, n = tot + float(loss), n + 1
        compressor.eval()
        vtot = vacc = vn = 0.0
        with torch.no_grad():
            for batch in val_batches:
                loss, acc = run(batch, False)
                vtot, vacc, vn = vtot + float(loss), vacc + acc, vn + 1
        val = vtot / max(1.0, vn)
        sched.step(val)
        history.append({"epoch": epoch, "train_loss": tot / max(1.0, n), "val_loss": val,
                        "val_acc": vacc / max(1.0, vn), "lr": opt.param_groups[0]["lr"]})
        save_compressor(compressor, last, epoch, opt, sched, val)
        if val < best_val:
            best_val = val
            save_compressor(compressor, best, epoch, opt, sched, val)
    compressor.eval()
    return {"history": history, "best_val": best_val, "last": last, "best": best}


def _compress_with_grad(compressor: _CCMBase, kv, it_len):
    """`forward` of the modules is wrapped in no_grad for inference; training calls the layer path."""
    img = 0 if not hasattr(compressor, "compress_ik") else int(it_len[0])
    return [compressor.compress_layer_kv(k, v, l, img) for l, (k, v) in enumerate(kv)]
