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

import math
import os
from dataclasses import dataclass
from typing import Any, Callable, Dict, Iterable, List, Optional, Sequence, Tuple

import torch
import torch.nn.functional as F
from torch import nn

from .ccm import (KVCacheHybridCompressor, KVCacheLinearDecoupleCompressor, _CCMBase, load_compressor,
                  save_compressor)


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


    # ------------------------------------------------ probability-space interface
    # The reference's loss takes probability distributions and mixes its terms with
    # (alpha, beta, 1 - alpha - beta) (utils_ccm/module_ccm_v11.py:1281-1867).  The methods below give
    # that interface; `alpha`, `beta`, `epsilon`, `p_threshold` and the position weights are
    # attributes with the reference's defaults.
    alpha, beta, epsilon, p_threshold = 1.0, 1.0, 1e-8, 0.9
    high_weight_count, low_weight, high_weight = 30, 1.0, 3.0

    def _mix(self, target: torch.Tensor, mid: torch.Tensor, out: torch.Tensor,
             weights: Optional[torch.Tensor] = None) -> torch.Tensor:
        eps = self.epsilon
        ce_rows = -(target * torch.log(out + eps)).sum(-1)
        ce = (ce_rows * weights).mean() if weights is not None else ce_rows.mean()
        m = 0.5 * (mid + out)
        js = 0.5 * ((mid * torch.log(mid / (m + eps) + eps)).sum(-1) +
                    (out * torch.log(out / (m + eps) + eps)).sum(-1)).mean()
        l1 = (mid - out).abs().sum(-1).mean()
        return self.alpha * ce + self.beta * js + (1.0 - self.alpha - self.beta) * l1

    def _targets(self, mid_probs: torch.Tensor) -> torch.Tensor:
        if self.strategy == "logit":
            return mid_probs
        return F.one_hot(mid_probs.argmax(-1), mid_probs.shape[-1]).to(mid_probs.dtype)

    def prob_loss(self, mid_probs: torch.Tensor, output_probs: torch.Tensor) -> torch.Tensor:
        """CE + JS + L1 between the original-KV distribution `mid_probs` and the compressed-KV
        distribution `output_probs`; the CE target is the distribution itself (strategy "logit") or
        its arg-max (the label strategies)."""
        return self._mix(self._targets(mid_probs), mid_probs, output_probs)

    def loss_weight(self, mid_probs: torch.Tensor, output_probs: torch.Tensor) -> torch.Tensor:
        """`prob_loss` with the first `high_weight_count` positions of each sequence weighted
        `high_weight` : `low_weight` in the CE term (label strategies)."""
        if self.strategy == "logit":
            return self.prob_loss(mid_probs, output_probs)
        w = torch.full(output_probs.shape[:-1], self.low_weight, device=output_probs.device)
        w[:, : self.high_weight_count] = self.high_weight
        return self._mix(self._targets(mid_probs), mid_probs, output_probs, w)

    def loss_gen(self, mid_probs: torch.Tensor, output_probs: torch.Tensor, gen_output_probs: torch.Tensor
                 ) -> torch.Tensor:
        """Teacher-forced loss plus the same loss on the free-running generation (cut to the shorter)."""
        n = min(mid_probs.shape[1], gen_output_probs.shape[1])
        return 0.5 * (self.prob_loss(mid_probs, output_probs) +
                      self.prob_loss(mid_probs[:, :n], gen_output_probs[:, :n]))

    @staticmethod
    def indices_to_mask(indices: torch.Tensor, hidden_dim: int, mask: Optional[torch.Tensor] = None
                        ) -> torch.Tensor:
        """[B, S] indices -> bool [B, S, hidden_dim] with mask[b, s, indices[b, s]] set (added to `mask`)."""
        if mask is None:
            mask = torch.zeros(*indices.shape, hidden_dim, dtype=torch.bool, device=indices.device)
        return mask.scatter_(-1, indices.long().unsqueeze(-1), True)

    def get_top_p_mask(self, probs: torch.Tensor) -> torch.Tensor:
        """Per position, the smallest set of most likely tokens whose mass reaches `p_threshold`."""
        sp, si = torch.sort(probs, dim=-1, descending=True)
        keep = torch.cumsum(sp, dim=-1) <= self.p_threshold
        crossing = keep.sum(-1).clamp_max(probs.shape[-1] - 1)        # the token that crosses the threshold
        keep = self.indices_to_mask(crossing, probs.shape[-1], keep)
        return torch.zeros_like(probs, dtype=torch.bool).scatter_(-1, si, keep)

    def forward_attn(self, original_twice_outputs_logits: torch.Tensor, compress_output_logits: torch.Tensor,
                     pos_len: Sequence[int], orig_hidden_states: Sequence[torch.Tensor],
                     compress_hidden_states: Sequence[torch.Tensor], attention_mask: Any = None) -> torch.Tensor:
        """Half output-distribution loss with top-p soft labels over the first `pos_len[0] + pos_len[1]`
        positions, half per-layer hidden-state loss (MSE + cosine distance of the softmaxed states,
        the embedding layer skipped).  Both inputs are probability distributions despite their names."""
        n = int(pos_len[0]) + int(pos_len[1])
        base, comp = original_twice_outputs_logits, compress_output_logits
        head = base[:, :n] * self.get_top_p_mask(base[:, :n]).to(base.dtype)
        labels = head / (head.sum(-1, keepdim=True) + self.epsilon)
        eps = self.epsilon
        ce = -(labels * torch.log(comp[:, :n] + eps)).sum(-1).mean()
        m = 0.5 * (base + comp)
        js = 0.5 * ((base * torch.log(base / (m + eps) + eps)).sum(-1) +
                    (comp * torch.log(comp / (m + eps) + eps)).sum(-1)).mean()
        l1 = (base - comp).abs().sum(-1).mean()
        layer = base.new_zeros(())
        for i, (o, c) in enumerate(zip(orig_hidden_states, compress_hidden_states)):
            if i == 0:
                continue
            po, pc = torch.softmax(o.float(), -1), torch.softmax(c.float(), -1)
            layer = layer + F.mse_loss(c.float(), o.float()) + \
                (1.0 - F.cosine_similarity(pc.flatten(0, -2), po.flatten(0, -2), dim=-1).mean())
        out = self.alpha * ce + self.beta * js + (1.0 - self.alpha - self.beta) * l1
        return 0.5 * out + 0.5 * (layer / 2)

    @staticmethod
    def cvt_hidden_states(hidden_states: Sequence[Sequence[torch.Tensor]]) -> Tuple[torch.Tensor, ...]:
        """`generate()`'s per-step tuples (step -> layer -> [B, 1, H]) to per-layer [B, steps, H]."""
        n_layers = len(hidden_states[0])
        return tuple(torch.cat([step[l][:, -1:, :] for step in hidden_states], dim=1) for l in range(n_layers))

    @staticmethod
    def compute_attention_patterns(query: torch.Tensor, key: torch.Tensor, value: torch.Tensor,
                                   attention_mask: Optional[torch.Tensor] = None
                                   ) -> Tuple[torch.Tensor, torch.Tensor]:
        """softmax(Q K^T / sqrt(d)) (+ additive mask) and its product with V."""
        w = query @ key.transpose(-1, -2) / math.sqrt(query.shape[-1])
        if attention_mask is not None:
            w = w + attention_mask
        w = torch.softmax(w.float(), dim=-1).to(value.dtype)
        return w, w @ value

    @staticmethod
    def calc_metrics(mid_probs: torch.Tensor, output_probs: torch.Tensor):
        a, b = mid_probs.argmax(-1), output_probs.argmax(-1)
        return (a == b).float().mean(), a, b

    def calc_metrics2(self, mid_probs, output_probs, gen_output_probs):
        """Agreement of the teacher-forced and of the free-running predictions with the original ones."""
        a, b = mid_probs.argmax(-1), output_probs.argmax(-1)
        n = min(mid_probs.shape[1], gen_output_probs.shape[1])
        g = gen_output_probs[:, :n].argmax(-1)
        return (a == b).float().mean(), (a[:, :n] == g).float().mean(), a, b, g

    def calc_metrics3(self, mid_probs, output_probs):
        """Accuracy, mean length of a matching run, perplexity of the compressed model on the labels."""
        from .research import count_true_segments_with_zeros
        a, b = mid_probs.argmax(-1), output_probs.argmax(-1)
        runs = count_true_segments_with_zeros((a == b).reshape(-1))
        labels = F.one_hot(a, mid_probs.shape[-1]).to(output_probs.dtype)
        ce = -(labels * torch.log(output_probs + self.epsilon)).sum(-1).mean()
        return (a == b).float().mean(), float(sum(runs)) / len(runs), torch.exp(ce), a, b

    def calc_metrics4(self, mid_probs, output_probs, dmodel_probs):
        """As `calc_metrics3` for two candidate models and for "either of them is right"."""
        from .research import count_true_segments_with_zeros
        a = mid_probs.argmax(-1)
        e1, e2 = a == output_probs.argmax(-1), a == dmodel_probs.argmax(-1)
        e3 = e1 | e2
        run = lambda e: (lambda r: float(sum(r)) / (len(r) + 1e-5))(count_true_segments_with_zeros(e.reshape(-1)))  # noqa: E731
        return (e1.float().mean().item(), e2.float().mean().item(), e3.float().mean().item(),
                run(e1), run(e2), run(e3))


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
            tot, n = tot + float(loss.detach()), n + 1
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


# --------------------------------------------------------------------------- named recipes
def hf_forward_with_kv(model: Any, prefix_len_of: Callable[[Any], int]) -> Callable:
    """`forward_with_kv` for a HuggingFace-style causal LM (`model(input_ids=..., past_key_values=...,
    output_hidden_states=True, use_cache=True)`).  A batch is a dict with `input_ids` [B, T] (and
    whatever else the model takes); the first `prefix_len_of(batch)` tokens are the prefix whose KV
    is compressed, the rest is the continuation that is scored."""

    def as_pairs(past) -> List[Tuple[torch.Tensor, torch.Tensor]]:
        if hasattr(past, "to_legacy_cache"):
            past = past.to_legacy_cache()
        return [(k, v) for k, v in past]

    def fwd(batch: Dict[str, Any], kv: Optional[List[Tuple[torch.Tensor, torch.Tensor]]]):
        ids = batch["input_ids"]
        n = int(prefix_len_of(batch))
        extra = {k: v for k, v in batch.items() if k not in ("input_ids", "labels", "it_len")}
        if kv is None:
            out = model(input_ids=ids[:, :n], use_cache=True, output_hidden_states=True, **extra)
            return out.logits, tuple(out.hidden_states), as_pairs(out.past_key_values)
        past = tuple((k, v) for k, v in kv)
        out = model(input_ids=ids[:, n:], past_key_values=past, use_cache=True, output_hidden_states=True)
        return out.logits, tuple(out.hidden_states), as_pairs(out.past_key_values)

    return fwd


def _split(samples: Sequence[Any], train_ratio: float) -> Tuple[List[Any], List[Any]]:
    cut = max(1, min(len(samples) - 1, int(len(samples) * train_ratio))) if len(samples) > 1 else len(samples)
    return list(samples[:cut]), list(samples[cut:]) or list(samples[:cut])


def _recipe(cls, model: Any, samples: Sequence[Any], model_config: Any, forward_with_kv: Optional[Callable],
            prefix_len_of: Callable[[Any], int], it_len_of: Callable[[Any], Sequence[int]],
            compressor_load_path: str, compressor_save_name: str, out_dir: str, num_epochs: int,
            learning_rate: float, compression_ratio: int, train_ratio: float, is_continue: bool,
            strategy: str) -> Tuple[_CCMBase, Dict[str, Any]]:
    cfg_obj = model_config if model_config is not None else getattr(model, "config", None)
    if compressor_load_path:
        comp = load_compressor(compressor_load_path, src_config=cfg_obj, compression_factor=compression_ratio,
                               min_seq_len=2, kind="hybrid" if cls is KVCacheHybridCompressor else "decouple")
    else:
        comp = cls(cfg_obj, compression_ratio, 2)
    first = next(iter(model.parameters()), None) if hasattr(model, "parameters") else None
    if first is not None:
        comp = comp.to(first.device)
    fwd = forward_with_kv or hf_forward_with_kv(model, prefix_len_of)
    train, val = _split(samples, train_ratio)
    cfg = FinetuneConfig(lr=learning_rate, epochs=num_epochs, compression_factor=compression_ratio,
                         out_dir=out_dir, name=compressor_save_name, is_continue=is_continue)
    return comp, finetune_compressor(comp, fwd, train, val, cfg, it_len_of, KVCacheCompressionLoss(strategy))


def finetune_llava(model: Any, samples: Sequence[Any], model_config: Any = None,
                   forward_with_kv: Optional[Callable] = None,
                   prefix_len_of: Callable[[Any], int] = lambda b: int(b["it_len"][0]) + int(b["it_len"][1]),
                   it_len_of: Callable[[Any], Sequence[int]] = lambda b: b["it_len"],
                   compressor_load_path: str = "", compressor_save_name: str = "finetune_mlp_llava",
                   out_dir: str = "ckpt", num_epochs: int = 40, learning_rate: float = 5e-4,
                   compression_ratio: int = 5, train_ratio: float = 0.8, is_continue: bool = False,
                   strategy: str = "logit") -> Tuple[_CCMBase, Dict[str, Any]]:
    """The LLaVA recipe (scripts/finetune_llava.py:509-791): image / text decoupled compressor,
    Adam 5e-4, plateau scheduler, factor 5, 40 epochs, 80 / 20 split, `last_` / `best_` files."""
    return _recipe(KVCacheLinearDecoupleCompressor, model, samples, model_config, forward_with_kv, prefix_len_of,
                   it_len_of, compressor_load_path, compressor_save_name, out_dir, num_epochs, learning_rate,
                   compression_ratio, train_ratio, is_continue, strategy)


def finetune_com_minicpm(model: Any, samples: Sequence[Any], model_config: Any = None,
                         forward_with_kv: Optional[Callable] = None,
                         prefix_len_of: Callable[[Any], int] = lambda b: int(b["it_len"][0]) + int(b["it_len"][1]),
                         it_len_of: Callable[[Any], Sequence[int]] = lambda b: (0, int(sum(b["it_len"]))),
                         compressor_load_path: str = "", compressor_save_name: str = "finetune_mlp_minicpm",
                         out_dir: str = "ckpt", num_epochs: int = 40, learning_rate: float = 5e-4,
                         compression_ratio: int = 5, train_ratio: float = 0.8, is_continue: bool = False,
                         strategy: str = "logit") -> Tuple[_CCMBase, Dict[str, Any]]:
    """The MiniCPM recipe (scripts/finetune_minicpm.py:863-1195, defaults :1408-1445): the hybrid
    compressor (text banks only; the whole prefix counts as text), otherwise as for LLaVA."""
    return _recipe(KVCacheHybridCompressor, model, samples, model_config, forward_with_kv, prefix_len_of,
                   it_len_of, compressor_load_path, compressor_save_name, out_dir, num_epochs, learning_rate,
                   compression_ratio, train_ratio, is_continue, strategy)


# ------------------------------------------------------------- script-level helpers
# Helper names of the reference's fine-tuning scripts (scripts/finetune_llava.py:29-81, :237-250, :948-951;
# scripts/finetune_minicpm.py:118-123, :254-265, :785-860).
def set_seed(seed: int) -> None:
    import random
    random.seed(seed)
    torch.manual_seed(seed)
    if torch.cuda.is_available():
        torch.cuda.manual_seed_all(seed)


def save_checkpoint(epoch: int, model: _CCMBase, optimizer: Any, scheduler: Any, loss: float, is_best: bool,
                    filefoldname: str = "ckpt_store", filename: str = "checkpoint.pth") -> str:
    """`last_<filename>` always, `best_<filename>` when `is_best`; the layout of `save_compressor`."""
    os.makedirs(filefoldname, exist_ok=True)
    last = os.path.join(filefoldname, f"last_{filename}")
    save_compressor(model, last, epoch, optimizer, scheduler, loss)
    if is_best:
        save_compressor(model, os.path.join(filefoldname, f"best_{filename}"), epoch, optimizer, scheduler, loss)
    return last


def load_checkpoint(model: _CCMBase, optimizer: Any = None, scheduler: Any = None,
                    filename: str = "checkpoint.pth") -> Tuple[int, float]:
    """Restore compressor, optimizer and scheduler; returns (epoch, loss), or (0, inf) without a file."""
    if not os.path.isfile(filename):
        return 0, float("inf")
    blob = torch.load(filename, map_location="cpu", weights_only=False)
    state = blob["model_state_dict"]
    model.load_state_dict(state.get("compressor", state))
    if optimizer is not None and blob.get("optimizer_state_dict"):
        optimizer.load_state_dict(blob["optimizer_state_dict"])
    if scheduler is not None and blob.get("scheduler_state_dict"):
        scheduler.load_state_dict(blob["scheduler_state_dict"])
    return int(blob.get("epoch", 0)), float(blob.get("loss", float("inf")))


def load_finetune_compressor(compressor_path: str, src_config: Any = None, device: Any = None) -> _CCMBase:
    """The compressor class that matches the file, with its weights, in eval mode on `device`."""
    m = load_compressor(compressor_path, src_config=src_config)
    return (m.to(device) if device is not None else m).eval()


def parse_string_with_image(text: str, special_token: str = "<image>") -> Tuple[str, int]:
    """(text without the image marker, 1 if the marker was there else 0)."""
    if special_token in text:
        return text.replace(special_token, "").strip(), 1
    return text, 0


def load_text_data(json_path: str, num_samples: int, seed: Optional[int] = None) -> List[str]:
    """First human turn of every conversation of a ShareGPT / LLaVA-style JSON, whitespace-normalised,
    shuffled; `num_samples` < 0 keeps all."""
    import json
    import random
    with open(json_path, "r", encoding="utf-8") as fh:
        data = json.load(fh)
    texts = [" ".join(d["conversations"][0]["value"].split()) for d in data
             if d.get("conversations") and d["conversations"][0].get("from") == "human"]
    random.Random(seed).shuffle(texts)
    return texts if num_samples < 0 else texts[:num_samples]


@torch.no_grad()
def validate(compressor: _CCMBase, forward_with_kv: Callable, val_batches: Iterable[Any],
             it_len_of: Callable[[Any], Sequence[int]] = lambda b: (0, 0),
             loss_fn: Optional[KVCacheCompressionLoss] = None) -> Tuple[float, float]:
    """(mean loss, mean agreement with the original-KV predictions) over `val_batches`."""
    loss_fn = loss_fn or KVCacheCompressionLoss("logit")
    compressor.eval()
    tot = acc = n = 0.0
    for batch in val_batches:
        _, _, kv = forward_with_kv(batch, None)
        t_logits, t_hidden, _ = forward_with_kv(batch, kv)
        s_logits, s_hidden, _ = forward_with_kv(batch, compressor(kv, it_len_of(batch)))
        loss, _ = loss_fn(s_logits, t_logits, None, s_hidden, t_hidden)
        tot, acc, n = tot + float(loss), acc + loss_fn.accuracy(s_logits, t_logits), n + 1
    return tot / max(1.0, n), acc / max(1.0, n)


validate_llava = validate_minicpm = validate
finetune_com = finetune_llava


def main(argv: Optional[Sequence[str]] = None) -> Dict[str, Any]:
    """`python -m fastcache_b200.compress.train --model-path DIR --data FILE.json ...` fine-tunes a
    compressor for a HuggingFace checkpoint.  Samples come from the dataset loaders of
    `fastcache_b200.serving.datasets`; this entry distils on the text of each conversation (question and
    reference answers), the first half as the prefix whose KV is compressed."""
    import argparse
    import random

    ap = argparse.ArgumentParser(description="fine-tune a CCM merge compressor by distillation")
    ap.add_argument("--model-path", required=True)
    ap.add_argument("--data", required=True, help="llava_v1_5_mix665k-style JSON")
    ap.add_argument("--images", default="", help="folder the JSON's image paths are relative to")
    ap.add_argument("--datasets-type", default="image", choices=["text", "image"])
    ap.add_argument("--model-mode", default="minicpm", choices=["llava", "minicpm"])
    ap.add_argument("--num-samples", type=int, default=320)
    ap.add_argument("--max-input-len", type=int, default=512)
    ap.add_argument("--epochs", type=int, default=40)
    ap.add_argument("--lr", type=float, default=5e-4)
    ap.add_argument("--compression-ratio", type=int, default=5)
    ap.add_argument("--train-ratio", type=float, default=0.8)
    ap.add_argument("--compressor-load-path", default="")
    ap.add_argument("--compressor-save-name", default="")
    ap.add_argument("--out-dir", default="ckpt")
    ap.add_argument("--continue", dest="is_continue", action="store_true")
    ap.add_argument("--seed", type=int, default=48)
    a = ap.parse_args(argv)

    from transformers import AutoModelForCausalLM, AutoTokenizer
    from ..serving.datasets import load_image_data

    random.seed(a.seed)
    torch.manual_seed(a.seed)
    tok = AutoTokenizer.from_pretrained(a.model_path, trust_remote_code=True)
    model = AutoModelForCausalLM.from_pretrained(a.model_path, trust_remote_code=True,
                                                 torch_dtype=torch.bfloat16).eval()
    if torch.cuda.is_available():
        model = model.cuda()
    for p_ in model.parameters():
        p_.requires_grad_(False)
    dev = next(model.parameters()).device
    samples = []
    for rec in load_image_data(a.data, a.images, a.num_samples, seed=a.seed):
        ids = tok(rec.prompt + " " + " ".join(rec.answers), return_tensors="pt", truncation=True,
                  max_length=a.max_input_len)["input_ids"].to(dev)
        if ids.shape[1] < 4 * a.compression_ratio:
            continue
        half = ids.shape[1] // 2
        samples.append({"input_ids": ids, "it_len": (0, half)})
    fn = finetune_llava if a.model_mode == "llava" else finetune_com_minicpm
    name = a.compressor_save_name or f"finetune_mlp_{a.model_mode}"
    _, result = fn(model, samples, compressor_load_path=a.compressor_load_path, compressor_save_name=name,
                   out_dir=a.out_dir, num_epochs=a.epochs, learning_rate=a.lr,
                   compression_ratio=a.compression_ratio, train_ratio=a.train_ratio, is_continue=a.is_continue)
    print({k: result[k] for k in ("best_val", "last", "best")})
    return result


if __name__ == "__main__":
    main()
