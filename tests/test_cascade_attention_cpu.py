"""Shared-prefix (cascade) attention: requests that start with the same cached blocks attend
to them in one pass; tokens must equal those of the ordinary path."""
import torch

from vllm_gcu_b200.engine.llm import LLM
from vllm_gcu_b200.engine.request import SamplingParams
from vllm_gcu_b200.layers.attention import cascade_attention
from vllm_gcu_b200.ops import ref


def test_cascade_equals_full_attention_on_the_reference_ops():
    g = torch.Generator().manual_seed(0)
    nb, bs, Hq, Hkv, D = 24, 16, 4, 2, 64
    kc = torch.randn(nb, bs, Hkv, D, generator=g)
    vc = torch.randn(nb, bs, Hkv, D, generator=g)
    prefix_blocks = [3, 7]                          # 32 shared tokens
    bt = torch.tensor([prefix_blocks + [10, 11], prefix_blocks + [12, 0], prefix_blocks + [13, 14]],
                      dtype=torch.int32)
    seq_lens = torch.tensor([32 + 20, 32 + 1, 32 + 9], dtype=torch.int32)
    q_lens = [5, 1, 9]
    cu = torch.tensor([0, 5, 6, 15], dtype=torch.int32)
    q = torch.randn(15, Hq, D, generator=g)
    want = ref.varlen_prefill_attention(q, kc, vc, bt, cu, seq_lens, D ** -0.5)
    got = cascade_attention(q, kc, vc, bt, cu, seq_lens, D ** -0.5, 32, q_lens, native=False)
    assert (got - want).abs().max().item() < 1e-5


def _run(cascade_min):
    llm = LLM("tiny-llama", device="cpu", block_size=16, max_num_seqs=8, max_num_batched_tokens=256,
              max_model_len=256, num_gpu_blocks=128, dtype="float32",
              additional_config={"cascade_min_tokens": cascade_min})
    g = torch.Generator().manual_seed(1)
    shared = torch.randint(0, 32000, (64,), generator=g).tolist()
    tails = [torch.randint(0, 32000, (n,), generator=g).tolist() for n in (5, 9, 1, 12)]
    sp = SamplingParams(max_tokens=6, temperature=0.0, ignore_eos=True)
    llm.generate([shared + [7]], sp)                # fills the prefix cache
    outs = llm.generate([shared + t for t in tails], sp)
    return llm, [o.outputs[0].token_ids for o in outs]


def test_engine_uses_cascade_for_a_shared_cached_prefix():
    plain_llm, plain = _run(0)
    casc_llm, casc = _run(32)
    assert plain_llm.engine.runner.cascade_steps == 0
    assert casc_llm.engine.runner.cascade_steps > 0
    assert plain == casc
