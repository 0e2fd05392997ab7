"""Preemption through the engine on the CPU path: with too few KV blocks for the batch the
scheduler preempts; by recomputation (default) and by swapping to host blocks
(``num_cpu_blocks`` > 0) the generated tokens must equal those of an engine with ample cache."""
import torch

from vllm_gcu_b200.engine.llm import LLM
from vllm_gcu_b200.engine.request import SamplingParams


def _run(num_blocks, cpu_blocks, prefix):
    llm = LLM("tiny-llama", device="cpu", max_num_seqs=4, max_num_batched_tokens=64,
              max_model_len=256, num_gpu_blocks=num_blocks, num_cpu_blocks=cpu_blocks,
              dtype="float32", enable_prefix_caching=prefix)
    g = torch.Generator().manual_seed(7)
    prompts = [torch.randint(0, 32000, (n,), generator=g).tolist() for n in (50, 44, 37)]
    sp = SamplingParams(max_tokens=30, temperature=0.0, ignore_eos=True)
    outs = llm.generate(prompts, sp)
    return [o.outputs[0].token_ids for o in outs], llm.engine.scheduler


def test_swap_and_recompute_preemption_reproduce_the_unpreempted_tokens():
    want, s0 = _run(64, 0, False)
    assert s0.num_preemptions == 0
    got_r, s1 = _run(12, 0, False)                # 3 x ~5 blocks do not fit in 12
    assert s1.num_preemptions > 0 and s1.num_swaps == 0
    assert got_r == want
    got_s, s2 = _run(12, 16, False)
    assert s2.num_swaps > 0
    assert got_s == want
    assert sorted(s2.cpu_free) == list(range(16))
    got_p, s3 = _run(12, 16, True)                # with the prefix cache holding freed blocks
    assert s3.num_swaps > 0 and got_p == want
