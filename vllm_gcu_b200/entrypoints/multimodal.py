"""Images in chat requests: from OpenAI-style message parts to engine inputs.

A chat message's ``content`` may be a list of parts, ``{"type": "text", "text": ...}`` and
``{"type": "image_url", "image_url": {"url": "data:image/png;base64,..."}}`` (a local file path
or ``file://`` URL also works; there is no network access from the server).  Two ways lead from
there to ``(prompt_token_ids, multi_modal_data)``:

* ``HFProcessorAdapter``: the checkpoint's own HuggingFace processor renders the chat template,
  expands the image placeholders and produces ``pixel_values`` with ``image_grid_thw`` /
  ``image_sizes`` (Qwen2-VL, Qwen2.5-VL, GLM-4.1V, LLaVA, LLaVA-NeXT, InternVL in the
  transformers layout, GOT-OCR-2.0): what the reference gets from vLLM's multimodal registry
  (vllm_gcu/models/got_ocr2/got_ocr2.py:600-819 registers such a processor for its own model);
* ``ModelProcessorAdapter``: models of this package that tile images themselves
  (``prepare_images`` of DeepSeek-VL2 and InternVL in its original layout): the text is
  tokenised with one placeholder per image and the model expands it.
"""
from __future__ import annotations

import base64
import io
from typing import Any, Optional, Sequence


def load_image(url: str):
    """PIL image (RGB) from a ``data:`` URL, a ``file://`` URL or a local path."""
    from PIL import Image
    if url.startswith("data:"):
        head, _, payload = url.partition(",")
        raw = base64.b64decode(payload) if ";base64" in head else payload.encode()
        return Image.open(io.BytesIO(raw)).convert("RGB")
    if url.startswith(("http://", "https://")):
        raise ValueError("remote image URLs are not fetched; send a data: URL")
    path = url[len("file://"):] if url.startswith("file://") else url
    return Image.open(path).convert("RGB")


def split_messages(messages: Sequence[dict]) -> tuple[list[dict], list]:
    """(messages with their image parts kept as ``{"type": "image"}`` markers, images in
    order of appearance)."""
    out, images = [], []
    for m in messages:
        content = m.get("content")
        if isinstance(content, list):
            parts = []
            for part in content:
                kind = part.get("type")
                if kind == "image_url":
                    ref_ = part.get("image_url")
                    images.append(load_image(ref_["url"] if isinstance(ref_, dict) else ref_))
                    parts.append({"type": "image"})
                elif kind == "image":
                    if "image" in part:
                        images.append(part["image"])
                    parts.append({"type": "image"})
                elif kind == "text":
                    parts.append({"type": "text", "text": part.get("text", "")})
                else:
                    raise ValueError(f"unsupported content part {kind!r}")
            out.append({**m, "content": parts})
        else:
            out.append(m)
    return out, images


class HFProcessorAdapter:
    """Wraps a HuggingFace processor (``AutoProcessor.from_pretrained(checkpoint)``)."""

    #: processor outputs the engine's ``prepare_request`` hooks understand
    KEYS = ("pixel_values", "image_grid_thw", "image_sizes", "images_spatial_crop")

    def __init__(self, processor: Any):
        self.processor = processor

    def __call__(self, messages: Sequence[dict], images: Sequence) -> tuple[list[int], dict]:
        text = self.processor.apply_chat_template(list(messages), add_generation_prompt=True,
                                                  tokenize=False)
        return self.from_text(text, images)

    def from_text(self, text: str, images: Sequence) -> tuple[list[int], dict]:
        """A prompt that already carries the model's image placeholders (the offline form:
        ``{"prompt": "<image>\\nDescribe.", "multi_modal_data": {"image": pil_image}}``)."""
        enc = self.processor(text=[text], images=list(images) or None, return_tensors="pt")
        ids = [int(t) for t in enc["input_ids"][0]]
        mm = {k: enc[k] for k in self.KEYS if k in enc}
        if "pixel_values" in mm and mm["pixel_values"].dim() == 5:
            mm["pixel_values"] = mm["pixel_values"][0]        # [1, views, ...] -> [views, ...]
        return ids, mm


class ModelProcessorAdapter:
    """For models with their own ``prepare_images(images, prompt_token_ids)``: the transcript is
    tokenised with one placeholder token where every image stands."""

    def __init__(self, model: Any, tokenizer: Any):
        self.model, self.tokenizer = model, tokenizer

    def __call__(self, messages: Sequence[dict], images: Sequence) -> tuple[list[int], dict]:
        import numpy as np
        import torch
        ids: list[int] = []
        for m in messages:
            ids += list(self.tokenizer.encode(f"{m.get('role', 'user')}: "))
            content = m.get("content")
            parts = content if isinstance(content, list) else [{"type": "text", "text": content}]
            for part in parts:
                if part.get("type") == "image":
                    ids.append(int(self.model.image_token_id))
                else:
                    ids += list(self.tokenizer.encode(part.get("text") or ""))
            ids += list(self.tokenizer.encode("\n"))
        ids += list(self.tokenizer.encode("assistant: "))
        tensors = [torch.from_numpy(np.asarray(im, dtype=np.float32) / 255.0).permute(2, 0, 1)
                   for im in images]
        return self.model.prepare_images(tensors, ids)


def default_processor(model_path: Optional[str], model: Any, tokenizer: Any):
    """The checkpoint's HuggingFace processor when it has one, else the model's own tiling,
    else None (text-only serving)."""
    if model_path:
        try:
            from transformers import AutoProcessor
            proc = AutoProcessor.from_pretrained(model_path)
            if hasattr(proc, "image_processor"):
                return HFProcessorAdapter(proc)
        except Exception:  # noqa: BLE001 - no processor files next to the checkpoint
            pass
    if model is not None and hasattr(model, "prepare_images"):
        return ModelProcessorAdapter(model, tokenizer)
    return None
