"""Datasets and the model holder of the compressor fine-tuning scripts.

Parity: utils_ccm/module_ccm_v11.py:16-33 (`LLM`: HuggingFace model + processor on the available
device), :129-181 (`CustomDataset`: one tokenised conversation per item, optionally also with a
second tokenizer), :183-252 (`CustomImageTextDataset`: processor-encoded image + text turns) and
:254-331 (`CustomImageTextMinicpmDataset`: the same for MiniCPM-V, with the input embeddings
already merged with the image features).

A conversation for the image datasets is the pair `(turns, kinds)` the reference's loaders build:
`turns[i] = (text, image)` and `kinds[i] == 1` marks a turn that carries an image.  Like the
reference, an item stops at the first turn without an image (multi-round text is not used for
training).
"""
from __future__ import annotations

from typing import Any, Dict, List, Sequence

import torch
from torch.utils.data import Dataset


class LLM:
    """HuggingFace vision-language model and its processor, in eval mode on the GPU when there is one."""

    def __init__(self, model_path: str, trust_remote_code: bool = True, processor_path: str | None = None,
                 torch_dtype: torch.dtype = torch.float32, model_cls: Any = None):
        from transformers import AutoProcessor
        if model_cls is None:
            from transformers import LlavaForConditionalGeneration as model_cls
        self.device = torch.device("cuda" if torch.cuda.is_available() else "cpu")
        self.torch_dtype = torch_dtype
        self.model = model_cls.from_pretrained(model_path, trust_remote_code=trust_remote_code,
                                               torch_dtype=torch_dtype).eval().to(self.device)
        self.processor = AutoProcessor.from_pretrained(processor_path or model_path,
                                                       trust_remote_code=trust_remote_code)


def _squeeze(enc: Dict[str, Any], keys: Sequence[str]) -> Dict[str, torch.Tensor]:
    return {k: enc[k].squeeze(0) for k in keys}


class CustomDataset(Dataset):
    def __init__(self, conversations: List[str], tokenizer: Any, max_length: int = 512):
        self.conversations, self.tokenizer, self.max_length = conversations, tokenizer, max_length
        self.tokenizer_draft: Any = None

    def new_tokenizer(self, tokenizer: Any) -> None:
        """Also encode every item with a second tokenizer (padded to `max_length`)."""
        self.tokenizer_draft = tokenizer

    def __len__(self) -> int:
        return len(self.conversations)

    def __getitem__(self, idx: int) -> Dict[str, torch.Tensor]:
        text = self.conversations[idx]
        enc = self.tokenizer(text, truncation=True, max_length=self.max_length, return_tensors="pt")
        out = _squeeze(enc, ("input_ids", "attention_mask"))
        if self.tokenizer_draft is not None:
            d = self.tokenizer_draft(text, truncation=True, padding="max_length", max_length=self.max_length,
                                     return_tensors="pt")
            out["draft_input_ids"] = d["input_ids"].squeeze(0)
            out["draft_attention_mask"] = d["attention_mask"].squeeze(0)
        return out


class CustomImageTextDataset(Dataset):
    def __init__(self, conversations: List[Any], processor: Any, max_length: int = 512,
                 launch_padding_flag: bool = True):
        self.conversations, self.processor = conversations, processor
        self.max_length, self.launch_padding_flag = max_length, launch_padding_flag

    def __len__(self) -> int:
        return len(self.conversations)

    def _pad_kw(self) -> Dict[str, Any]:
        kw: Dict[str, Any] = {"truncation": True, "return_tensors": "pt"}
        if self.launch_padding_flag:
            kw.update(padding="max_length", max_length=self.max_length)
        return kw

    def _encode(self, text: Any, image: Any) -> Dict[str, torch.Tensor]:
        enc = self.processor(images=image, text=text, **self._pad_kw())
        out = _squeeze(enc, ("input_ids", "attention_mask", "pixel_values"))
        out["type"] = torch.tensor([1.0])
        return out

    def __getitem__(self, idx: int) -> List[Dict[str, torch.Tensor]]:
        turns, kinds = self.conversations[idx][0], self.conversations[idx][1]
        items: List[Dict[str, torch.Tensor]] = []
        for (text, image), kind in zip(turns, kinds):
            if kind != 1:
                break
            items.append(self._encode(text, image))
        return items


class CustomImageTextMinicpmDataset(CustomImageTextDataset):
    """`model_runner` is the MiniCPM model (anything with `get_vllm_embedding` and `.device`)."""

    def __init__(self, conversations: List[Any], model_runner: Any, processor: Any, max_length: int = 512,
                 launch_padding_flag: bool = True):
        super().__init__(conversations, processor, max_length, launch_padding_flag)
        self.model = model_runner

    def _encode(self, text: Any, image: Any) -> Dict[str, torch.Tensor]:
        prompt = self.processor.tokenizer.apply_chat_template(text, tokenize=False, add_generation_prompt=True)
        enc = self.processor([prompt], [image], **self._pad_kw())
        if hasattr(enc, "to"):
            enc = enc.to(getattr(self.model, "device", "cpu"))
        inputs = {k: enc[k] for k in ("input_ids", "attention_mask", "image_bound", "pixel_values", "tgt_sizes")}
        with torch.no_grad():
            embeds, _ = self.model.get_vllm_embedding(inputs)
        return {"input_ids": inputs["input_ids"].squeeze(0), "attention_mask": inputs["attention_mask"].squeeze(0),
                "inputs_embeds": embeds.squeeze(0), "pixel_values": inputs["pixel_values"],
                "type": torch.tensor([1.0])}
