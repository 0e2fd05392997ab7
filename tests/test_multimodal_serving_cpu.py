"""Images in chat requests on the CPU engine: a ``data:`` URL in the message parts reaches the
vision tower through the server (a processor in the HuggingFace call convention for LLaVA, the
model's own tiling for InternVL), with the same tokens as the offline engine on the same pixels;
the multi-process executor carries the tensors to its workers."""
import asyncio
import base64
import io

import pytest
import torch

from vllm_gcu_b200.config import CacheConfig, EngineConfig, ModelConfig, SchedulerConfig
from vllm_gcu_b200.engine.async_llm import AsyncLLM
from vllm_gcu_b200.engine.llm import LLM
from vllm_gcu_b200.engine.request import SamplingParams
from vllm_gcu_b200.entrypoints.api_server import ByteTokenizer, build_app
from vllm_gcu_b200.entrypoints.multimodal import (HFProcessorAdapter, ModelProcessorAdapter,
                                                  load_image, split_messages)

IMG = 290


def _png_url(seed: int, size=(40, 30)) -> str:
    from PIL import Image
    import numpy as np
    arr = np.random.default_rng(seed).integers(0, 255, (size[1], size[0], 3), dtype=np.uint8)
    buf = io.BytesIO()
    Image.fromarray(arr).save(buf, format="PNG")
    return "data:image/png;base64," + base64.b64encode(buf.getvalue()).decode()


def _llava_config() -> ModelConfig:
    d = {"architectures": ["LlavaForConditionalGeneration"],
         "text_config": dict(vocab_size=300, hidden_size=64, intermediate_size=128,
                             num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
                             max_position_embeddings=256, tie_word_embeddings=False,
                             rms_norm_eps=1e-6),
         "vision_config": dict(hidden_size=32, intermediate_size=64, num_hidden_layers=3,
                               num_attention_heads=2, image_size=28, patch_size=14,
                               hidden_act="quick_gelu"),
         "image_token_index": IMG, "vision_feature_layer": -2,
         "vision_feature_select_strategy": "default"}
    return ModelConfig.from_hf_dict(d, dtype=torch.float32)


class _Processor:
    """Stand-in with the call convention of a HuggingFace processor: chat template, placeholder
    expansion (4 rows per image), 28 x 28 pixel tensors."""
    image_processor = object()

    def apply_chat_template(self, messages, add_generation_prompt=True, tokenize=False):
        text = ""
        for m in messages:
            parts = m["content"] if isinstance(m["content"], list) else \
                [{"type": "text", "text": m["content"]}]
            text += "".join("<image>" if p["type"] == "image" else p["text"] for p in parts) + "\n"
        return text

    def __call__(self, text, images=None, return_tensors="pt"):
        import numpy as np
        ids = []
        for piece in text[0].split("<image>"):
            ids += [3 + b for b in piece.encode()] + [IMG] * 4
        ids = ids[:-4]
        px = [torch.from_numpy(np.asarray(im.resize((28, 28)), dtype=np.float32) / 127.5 - 1.0)
              .permute(2, 0, 1) for im in images or []]
        return {"input_ids": torch.tensor([ids]), "pixel_values": torch.stack(px)}


def test_message_parts_and_image_loading(tmp_path):
    url = _png_url(0)
    assert load_image(url).size == (40, 30)
    load_image(url).save(tmp_path / "a.png")
    assert load_image(str(tmp_path / "a.png")).size == (40, 30)
    assert load_image("file://" + str(tmp_path / "a.png")).size == (40, 30)
    with pytest.raises(ValueError):
        load_image("https://example.com/a.png")
    msgs, images = split_messages([
        {"role": "system", "content": "be brief"},
        {"role": "user", "content": [{"type": "text", "text": "what is "},
                                     {"type": "image_url", "image_url": {"url": url}},
                                     {"type": "text", "text": "?"}]}])
    assert len(images) == 1 and msgs[0]["content"] == "be brief"
    assert [p["type"] for p in msgs[1]["content"]] == ["text", "image", "text"]
    with pytest.raises(ValueError):
        split_messages([{"role": "user", "content": [{"type": "audio"}]}])


@pytest.mark.timeout(180)
def test_chat_with_an_image_matches_the_offline_engine():
    httpx = pytest.importorskip("httpx")
    mc = _llava_config()
    cfg = EngineConfig(model=mc, cache=CacheConfig(num_gpu_blocks=64),
                       scheduler=SchedulerConfig(max_num_seqs=4, max_num_batched_tokens=32,
                                                 max_model_len=128), device="cpu", seed=0)
    eng = AsyncLLM(cfg)
    adapter = HFProcessorAdapter(_Processor())
    app = build_app(eng, ByteTokenizer(300), "tiny-llava", mm_processor=adapter)
    url = _png_url(1)
    messages = [{"role": "user", "content": [{"type": "text", "text": "see "},
                                             {"type": "image_url", "image_url": {"url": url}},
                                             {"type": "text", "text": " ok"}]}]
    ids, mm = adapter(*split_messages(messages))
    assert ids.count(IMG) == 4 and mm["pixel_values"].shape == (1, 3, 28, 28)
    off = LLM(_llava_config(), device="cpu", max_num_seqs=4, max_num_batched_tokens=32,
              max_model_len=128, num_gpu_blocks=64, seed=0)
    sp = SamplingParams(max_tokens=5, temperature=0.0, ignore_eos=True)
    want = off.generate([{"prompt_token_ids": ids, "multi_modal_data": mm}], sp)[0]
    plain = off.generate([[t for t in ids if t != IMG]], sp)[0]
    assert want.outputs[0].token_ids != plain.outputs[0].token_ids

    async def run():
        transport = httpx.ASGITransport(app=app)
        async with httpx.AsyncClient(transport=transport, base_url="http://t") as c:
            body = {"messages": messages, "max_tokens": 5, "temperature": 0.0,
                    "ignore_eos": True}
            r = await c.post("/v1/chat/completions", json=body)
            assert r.status_code == 200, r.text
            text = r.json()["choices"][0]["message"]["content"]
            assert text == ByteTokenizer(300).decode(want.outputs[0].token_ids)
            bad = {**body, "messages": [{"role": "user", "content": [
                {"type": "image_url", "image_url": {"url": "https://example.com/x.png"}}]}]}
            assert (await c.post("/v1/chat/completions", json=bad)).status_code == 400
    try:
        asyncio.run(run())
    finally:
        eng.shutdown()


def test_model_side_tiling_adapter_builds_engine_inputs():
    """InternVL in its original layout tiles images itself: one placeholder per image in the
    transcript is expanded to the rows of that image's tiles."""
    d = {"architectures": ["InternVLChatModel"],
         "llm_config": dict(architectures=["Qwen2ForCausalLM"], vocab_size=300, hidden_size=64,
                            intermediate_size=128, num_hidden_layers=2, num_attention_heads=4,
                            num_key_value_heads=2, max_position_embeddings=512,
                            rms_norm_eps=1e-6, tie_word_embeddings=False),
         "vision_config": dict(hidden_size=32, intermediate_size=64, num_hidden_layers=2,
                               num_attention_heads=2, image_size=28, patch_size=7),
         "downsample_ratio": 0.5, "img_context_token_id": IMG, "max_dynamic_patch": 4}
    llm = LLM(ModelConfig.from_hf_dict(d, dtype=torch.float32), device="cpu", max_num_seqs=4,
              max_num_batched_tokens=64, max_model_len=256, num_gpu_blocks=64)
    adapter = ModelProcessorAdapter(llm.engine.model, ByteTokenizer(300))
    msgs, images = split_messages([{"role": "user", "content": [
        {"type": "image_url", "image_url": {"url": _png_url(2, size=(84, 28))}},
        {"type": "text", "text": "hi"}]}])
    ids, mm = adapter(msgs, images)
    tiles = mm["pixel_values"].shape[0]
    assert tiles == 4 and ids.count(IMG) == tiles * llm.engine.model.tokens_per_tile   # 3 + thumb
    out = llm.generate([{"prompt_token_ids": ids, "multi_modal_data": mm}],
                       SamplingParams(max_tokens=3, temperature=0.0, ignore_eos=True))
    assert len(out[0].outputs[0].token_ids) == 3


@pytest.mark.timeout(300)
def test_executor_carries_image_tensors_to_its_workers():
    from vllm_gcu_b200.config import ParallelConfig
    from vllm_gcu_b200.engine.executor import MultiprocExecutor
    cfg = EngineConfig(model=_llava_config(), cache=CacheConfig(num_gpu_blocks=64),
                       scheduler=SchedulerConfig(max_num_seqs=4, max_num_batched_tokens=32,
                                                 max_model_len=128),
                       parallel=ParallelConfig(tensor_parallel_size=2, comm_backend="nccl"),
                       device="cpu", seed=0)
    ids = [5, 6] + [IMG] * 4 + [7, 8]
    g = torch.Generator().manual_seed(0)
    px = [torch.randn(1, 3, 28, 28, generator=g) for _ in range(2)]
    sp = SamplingParams(max_tokens=5, temperature=0.0, ignore_eos=True)
    ex = MultiprocExecutor(cfg)
    try:
        rids = [ex.add_request(ids, sp, multi_modal_data={"pixel_values": p})
                for p in (px[0], px[1], px[0])]
        got = {}
        for _ in range(600):
            for o in ex.poll(0.1):
                if o.finished:
                    got[o.request_id] = o.outputs[0].token_ids
            if len(got) == 3:
                break
    finally:
        ex.shutdown()
    a, b, c = (got[r] for r in rids)
    assert len(a) == 5 and a == c and a != b       # the pixels decide the continuation


def test_offline_prompt_with_a_pil_image():
    """The offline form of upstream vLLM: a text prompt with the placeholder and the image as a
    PIL object; the processor expands and encodes it."""
    llm = LLM(_llava_config(), device="cpu", max_num_seqs=4, max_num_batched_tokens=32,
              max_model_len=128, num_gpu_blocks=64, seed=0,
              mm_processor=HFProcessorAdapter(_Processor()))
    img = load_image(_png_url(1))
    sp = SamplingParams(max_tokens=4, temperature=0.0, ignore_eos=True)
    a = llm.generate([{"prompt": "see <image> ok", "multi_modal_data": {"image": img}}], sp)[0]
    ids, mm = HFProcessorAdapter(_Processor()).from_text("see <image> ok", [img])
    b = llm.generate([{"prompt_token_ids": ids, "multi_modal_data": mm}], sp)[0]
    assert a.outputs[0].token_ids == b.outputs[0].token_ids and a.prompt_token_ids == ids
    with pytest.raises(ValueError):
        LLM(_llava_config(), device="cpu", max_num_seqs=4, max_num_batched_tokens=32,
            max_model_len=128, num_gpu_blocks=64).generate(
            [{"prompt": "x <image>", "multi_modal_data": {"image": img}}], sp)


def test_checkpoint_directory_with_a_huggingface_processor(tmp_path):
    """A LLaVA checkpoint directory as users have it (weights, tokenizer with an ``<image>``
    token and a chat template, image processor): ``LLM(directory)`` finds the processor, a text
    prompt with the placeholder and a PIL image gives the tokens of transformers' ``generate``
    on the processor's own encoding, and chat messages with an image part are expanded."""
    import numpy as np
    tr = pytest.importorskip("transformers")
    tokenizers = pytest.importorskip("tokenizers")
    from PIL import Image
    from tokenizers import Tokenizer, decoders, models, pre_tokenizers, trainers
    tok = Tokenizer(models.BPE(unk_token="<unk>"))
    tok.pre_tokenizer = pre_tokenizers.ByteLevel(add_prefix_space=False)
    tok.decoder = decoders.ByteLevel()
    tok.train_from_iterator(
        ["describe the picture please", "what is in this image?"] * 20,
        trainers.BpeTrainer(vocab_size=300,
                            special_tokens=["<unk>", "<s>", "</s>", "<image>", "<pad>"],
                            initial_alphabet=pre_tokenizers.ByteLevel.alphabet()))
    fast = tr.PreTrainedTokenizerFast(tokenizer_object=tok, bos_token="<s>", eos_token="</s>",
                                      unk_token="<unk>", pad_token="<pad>")
    fast.chat_template = ("{% for m in messages %}{{ m['role'] }}: {% for p in m['content'] %}"
                          "{% if p['type'] == 'image' %}<image>{% else %}{{ p['text'] }}"
                          "{% endif %}{% endfor %}\n{% endfor %}assistant: ")
    img_tok = fast.convert_tokens_to_ids("<image>")
    proc = tr.LlavaProcessor(
        image_processor=tr.CLIPImageProcessor(size={"shortest_edge": 28},
                                              crop_size={"height": 28, "width": 28}),
        tokenizer=fast, patch_size=14, vision_feature_select_strategy="default",
        image_token="<image>", num_additional_image_tokens=1)
    cfg = tr.LlavaConfig(
        text_config=dict(model_type="llama", vocab_size=len(fast), hidden_size=64,
                         intermediate_size=128, num_hidden_layers=2, num_attention_heads=4,
                         num_key_value_heads=2, max_position_embeddings=256,
                         tie_word_embeddings=False, rms_norm_eps=1e-6),
        vision_config=dict(model_type="clip_vision_model", hidden_size=32, intermediate_size=64,
                           num_hidden_layers=3, num_attention_heads=2, image_size=28,
                           patch_size=14, hidden_act="quick_gelu", projection_dim=16),
        image_token_index=img_tok, vision_feature_layer=-2,
        vision_feature_select_strategy="default", image_seq_length=4)
    torch.manual_seed(0)
    hf = tr.LlavaForConditionalGeneration(cfg).eval().float()
    d = str(tmp_path)
    hf.save_pretrained(d, safe_serialization=True)
    proc.save_pretrained(d)
    llm = LLM(d, device="cpu", max_num_seqs=4, max_num_batched_tokens=64, max_model_len=128,
              num_gpu_blocks=64, dtype="float32")
    assert isinstance(llm.mm_processor, HFProcessorAdapter)
    img = Image.fromarray(np.random.default_rng(0).integers(0, 255, (40, 52, 3), dtype=np.uint8))
    text = "<image>\ndescribe the picture"
    out = llm.generate([{"prompt": text, "multi_modal_data": {"image": img}}],
                       SamplingParams(max_tokens=5, temperature=0.0, ignore_eos=True))[0]
    enc = proc(text=[text], images=[img], return_tensors="pt")
    with torch.inference_mode():
        want = hf.generate(**enc, max_new_tokens=5, do_sample=False,
                           pad_token_id=0)[0, enc["input_ids"].shape[1]:].tolist()
    assert out.prompt_token_ids == enc["input_ids"][0].tolist()
    assert out.outputs[0].token_ids == want
    msgs, images = split_messages([{"role": "user", "content": [
        {"type": "image", "image": img}, {"type": "text", "text": "what is in this image?"}]}])
    ids, mm = llm.mm_processor(msgs, images)
    assert ids.count(img_tok) == 4 and tuple(mm["pixel_values"].shape) == (1, 3, 28, 28)


def test_qwen2_vl_checkpoint_directory_with_its_processor(tmp_path):
    """Qwen2-VL with the HuggingFace processor of its checkpoint directory: the processor
    resizes and patchifies the image and expands the placeholder; the engine's tokens equal
    transformers' ``generate`` on the same encoding (multimodal rotary positions included)."""
    import numpy as np
    tr = pytest.importorskip("transformers")
    pytest.importorskip("tokenizers")
    from PIL import Image
    from tokenizers import Tokenizer, decoders, models, pre_tokenizers, trainers
    tok = Tokenizer(models.BPE(unk_token="<unk>"))
    tok.pre_tokenizer = pre_tokenizers.ByteLevel(add_prefix_space=False)
    tok.decoder = decoders.ByteLevel()
    sp_toks = ["<unk>", "<|endoftext|>", "<|vision_start|>", "<|vision_end|>", "<|image_pad|>",
               "<|video_pad|>", "<|im_start|>", "<|im_end|>"]
    tok.train_from_iterator(
        ["describe the picture please", "what is in this image?"] * 20,
        trainers.BpeTrainer(vocab_size=300, special_tokens=sp_toks,
                            initial_alphabet=pre_tokenizers.ByteLevel.alphabet()))
    fast = tr.PreTrainedTokenizerFast(tokenizer_object=tok, eos_token="<|endoftext|>",
                                      unk_token="<unk>", pad_token="<|endoftext|>")
    fast.chat_template = (
        "{% for m in messages %}<|im_start|>{{ m['role'] }}\n{% for p in m['content'] %}"
        "{% if p['type'] == 'image' %}<|vision_start|><|image_pad|><|vision_end|>{% else %}"
        "{{ p['text'] }}{% endif %}{% endfor %}<|im_end|>\n{% endfor %}<|im_start|>assistant\n")
    ids = {t: fast.convert_tokens_to_ids(t) for t in sp_toks}
    ip = tr.Qwen2VLImageProcessor(min_pixels=28 * 28 * 4, max_pixels=28 * 28 * 16, patch_size=14,
                                  merge_size=2, temporal_patch_size=2)
    proc = tr.Qwen2VLProcessor(image_processor=ip, tokenizer=fast,
                               video_processor=tr.Qwen2VLVideoProcessor(),
                               chat_template=fast.chat_template)
    text = dict(vocab_size=len(fast), hidden_size=64, intermediate_size=128, num_hidden_layers=2,
                num_attention_heads=4, num_key_value_heads=2, max_position_embeddings=512,
                rope_theta=10000.0, rms_norm_eps=1e-6, tie_word_embeddings=False,
                rope_scaling={"type": "mrope", "mrope_section": [2, 3, 3]})
    vision = dict(depth=2, embed_dim=32, hidden_size=64, mlp_ratio=2, num_heads=2, in_channels=3,
                  patch_size=14, spatial_merge_size=2, temporal_patch_size=2)
    cfg = tr.Qwen2VLConfig(text_config=text, vision_config=vision,
                           image_token_id=ids["<|image_pad|>"],
                           video_token_id=ids["<|video_pad|>"],
                           vision_start_token_id=ids["<|vision_start|>"],
                           vision_end_token_id=ids["<|vision_end|>"])
    torch.manual_seed(0)
    hf = tr.Qwen2VLForConditionalGeneration(cfg).eval().float()
    d = str(tmp_path)
    hf.save_pretrained(d, safe_serialization=True)
    proc.save_pretrained(d)
    llm = LLM(d, device="cpu", max_num_seqs=4, max_num_batched_tokens=64, max_model_len=256,
              num_gpu_blocks=64, dtype="float32")
    assert isinstance(llm.mm_processor, HFProcessorAdapter)
    img = Image.fromarray(np.random.default_rng(0).integers(0, 255, (60, 90, 3), dtype=np.uint8))
    prompt = "<|vision_start|><|image_pad|><|vision_end|>describe the picture"
    out = llm.generate([{"prompt": prompt, "multi_modal_data": {"image": img}}],
                       SamplingParams(max_tokens=5, temperature=0.0, ignore_eos=True))[0]
    enc = proc(text=[prompt], images=[img], return_tensors="pt")
    with torch.inference_mode():
        want = hf.generate(**enc, max_new_tokens=5, do_sample=False,
                           pad_token_id=1)[0, enc["input_ids"].shape[1]:].tolist()
    assert out.prompt_token_ids == enc["input_ids"][0].tolist()
    assert out.outputs[0].token_ids == want


def test_glm4v_checkpoint_directory_with_its_processor(tmp_path):
    """GLM-4.1V with the HuggingFace processor of its checkpoint directory against
    transformers' ``generate`` (prefill and decode steps with multimodal rotary positions)."""
    import numpy as np
    tr = pytest.importorskip("transformers")
    pytest.importorskip("tokenizers")
    from PIL import Image
    from tokenizers import Tokenizer, decoders, models, pre_tokenizers, trainers
    tok = Tokenizer(models.BPE(unk_token="<unk>"))
    tok.pre_tokenizer = pre_tokenizers.ByteLevel(add_prefix_space=False)
    tok.decoder = decoders.ByteLevel()
    sp_toks = ["<unk>", "<|endoftext|>", "<|begin_of_image|>", "<|end_of_image|>", "<|image|>",
               "<|video|>", "<|begin_of_video|>", "<|end_of_video|>"]
    tok.train_from_iterator(
        ["describe the picture please"] * 20,
        trainers.BpeTrainer(vocab_size=300, special_tokens=sp_toks,
                            initial_alphabet=pre_tokenizers.ByteLevel.alphabet()))
    fast = tr.PreTrainedTokenizerFast(tokenizer_object=tok, eos_token="<|endoftext|>",
                                      unk_token="<unk>", pad_token="<|endoftext|>")
    fast.chat_template = "{% for m in messages %}{{ m['content'] }}{% endfor %}"
    ids = {t: fast.convert_tokens_to_ids(t) for t in sp_toks}
    ip = tr.Glm4vImageProcessor(size={"shortest_edge": 28 * 28 * 4, "longest_edge": 28 * 28 * 16},
                                patch_size=14, merge_size=2, temporal_patch_size=2)
    proc = tr.Glm4vProcessor(image_processor=ip, tokenizer=fast,
                             video_processor=tr.Glm4vVideoProcessor(),
                             chat_template=fast.chat_template)
    text = dict(vocab_size=len(fast), hidden_size=64, intermediate_size=128, num_hidden_layers=2,
                num_attention_heads=4, num_key_value_heads=2, max_position_embeddings=512,
                rms_norm_eps=1e-6, tie_word_embeddings=False, attention_bias=True, pad_token_id=1,
                rope_parameters={"rope_type": "default", "rope_theta": 10000.0,
                                 "mrope_section": [2, 1, 1], "partial_rotary_factor": 0.5})
    vision = dict(depth=2, hidden_size=32, intermediate_size=48, num_heads=2, in_channels=3,
                  image_size=56, patch_size=14, spatial_merge_size=2, temporal_patch_size=2,
                  out_hidden_size=64, rms_norm_eps=1e-5, attention_bias=True, hidden_act="silu")
    cfg = tr.Glm4vConfig(text_config=text, vision_config=vision, image_token_id=ids["<|image|>"],
                         video_token_id=ids["<|video|>"],
                         image_start_token_id=ids["<|begin_of_image|>"],
                         image_end_token_id=ids["<|end_of_image|>"])
    torch.manual_seed(0)
    hf = tr.Glm4vForConditionalGeneration(cfg).eval().float()
    d = str(tmp_path)
    hf.save_pretrained(d, safe_serialization=True)
    proc.save_pretrained(d)
    llm = LLM(d, device="cpu", max_num_seqs=4, max_num_batched_tokens=64, max_model_len=256,
              num_gpu_blocks=64, dtype="float32")
    assert isinstance(llm.mm_processor, HFProcessorAdapter)
    img = Image.fromarray(np.random.default_rng(0).integers(0, 255, (60, 90, 3), dtype=np.uint8))
    prompt = "<|begin_of_image|><|image|><|end_of_image|>describe the picture"
    out = llm.generate([{"prompt": prompt, "multi_modal_data": {"image": img}}],
                       SamplingParams(max_tokens=5, temperature=0.0, ignore_eos=True))[0]
    enc = proc(text=[prompt], images=[img], return_tensors="pt")
    with torch.inference_mode():
        want = hf.generate(**enc, max_new_tokens=5, do_sample=False,
                           pad_token_id=1)[0, enc["input_ids"].shape[1]:].tolist()
    assert out.outputs[0].token_ids == want


@pytest.mark.parametrize("size", [(40, 90), (90, 40), (50, 50)])
def test_llava_next_checkpoint_directory_with_its_processor(tmp_path, size):
    """LLaVA-NeXT with its HuggingFace processor (any-resolution views as a 5-D pixel tensor plus
    the original image size) for wide, tall and square images against transformers."""
    import numpy as np
    tr = pytest.importorskip("transformers")
    pytest.importorskip("tokenizers")
    from PIL import Image
    from tokenizers import Tokenizer, decoders, models, pre_tokenizers, trainers
    tok = Tokenizer(models.BPE(unk_token="<unk>"))
    tok.pre_tokenizer = pre_tokenizers.ByteLevel(add_prefix_space=False)
    tok.decoder = decoders.ByteLevel()
    tok.train_from_iterator(
        ["describe the picture please"] * 20,
        trainers.BpeTrainer(vocab_size=300,
                            special_tokens=["<unk>", "<s>", "</s>", "<image>", "<pad>"],
                            initial_alphabet=pre_tokenizers.ByteLevel.alphabet()))
    fast = tr.PreTrainedTokenizerFast(tokenizer_object=tok, bos_token="<s>", eos_token="</s>",
                                      unk_token="<unk>", pad_token="<pad>")
    fast.chat_template = "{% for m in messages %}{{ m['content'] }}{% endfor %}"
    img_tok = fast.convert_tokens_to_ids("<image>")
    pin = [[28, 56], [56, 28], [56, 56]]
    ip = tr.LlavaNextImageProcessor(size={"shortest_edge": 28},
                                    crop_size={"height": 28, "width": 28},
                                    image_grid_pinpoints=pin)
    proc = tr.LlavaNextProcessor(image_processor=ip, tokenizer=fast, patch_size=7,
                                 vision_feature_select_strategy="default", image_token="<image>",
                                 num_additional_image_tokens=1)
    cfg = tr.LlavaNextConfig(
        text_config=dict(model_type="llama", vocab_size=len(fast), hidden_size=64,
                         intermediate_size=128, num_hidden_layers=2, num_attention_heads=4,
                         num_key_value_heads=2, max_position_embeddings=512,
                         tie_word_embeddings=False, rms_norm_eps=1e-6),
        vision_config=dict(model_type="clip_vision_model", hidden_size=32, intermediate_size=64,
                           num_hidden_layers=3, num_attention_heads=2, image_size=28,
                           patch_size=7, hidden_act="quick_gelu", projection_dim=16),
        image_token_index=img_tok, vision_feature_layer=-2,
        vision_feature_select_strategy="default", image_grid_pinpoints=pin, image_seq_length=16)
    torch.manual_seed(0)
    hf = tr.LlavaNextForConditionalGeneration(cfg).eval().float()
    with torch.no_grad():
        hf.model.image_newline.copy_(torch.randn(64) * 0.5)
    d = str(tmp_path)
    hf.save_pretrained(d, safe_serialization=True)
    proc.save_pretrained(d)
    llm = LLM(d, device="cpu", max_num_seqs=4, max_num_batched_tokens=128, max_model_len=512,
              num_gpu_blocks=64, dtype="float32")
    img = Image.fromarray(np.random.default_rng(0).integers(0, 255, (*size, 3), dtype=np.uint8))
    prompt = "<image>\ndescribe the picture"
    enc = proc(text=[prompt], images=[img], return_tensors="pt")
    out = llm.generate([{"prompt": prompt, "multi_modal_data": {"image": img}}],
                       SamplingParams(max_tokens=4, temperature=0.0, ignore_eos=True))[0]
    with torch.inference_mode():
        want = hf.generate(**enc, max_new_tokens=4, do_sample=False,
                           pad_token_id=4)[0, enc["input_ids"].shape[1]:].tolist()
    assert out.prompt_token_ids == enc["input_ids"][0].tolist()
    assert out.outputs[0].token_ids == want
