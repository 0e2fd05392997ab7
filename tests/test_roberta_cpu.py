"""XLM-RoBERTa reranker / embedding model against the HuggingFace implementation."""
import pytest
import torch

from vllm_gcu_b200.models.roberta import (PoolingRunner, RobertaConfig, RobertaEmbeddingModel,
                                          XLMRobertaForSequenceClassification,
                                          roberta_position_ids)


def test_position_ids_skip_padding():
    ids = torch.tensor([0, 5, 6, 1, 1, 0, 7, 2])
    pos = roberta_position_ids(ids, [0, 5, 8], padding_idx=1)
    assert pos.tolist() == [2, 3, 4, 1, 1, 2, 3, 4]


def test_reranker_matches_transformers():
    tr = pytest.importorskip("transformers")
    hf_cfg = tr.XLMRobertaConfig(vocab_size=200, hidden_size=64, num_hidden_layers=2,
                                 num_attention_heads=4, intermediate_size=128,
                                 max_position_embeddings=66, type_vocab_size=1, num_labels=1,
                                 pad_token_id=1, hidden_dropout_prob=0.0,
                                 attention_probs_dropout_prob=0.0)
    torch.manual_seed(0)
    hf = tr.XLMRobertaForSequenceClassification(hf_cfg).eval()
    cfg = RobertaConfig.from_hf_dict(hf_cfg.to_dict(), dtype=torch.float32)
    ours = XLMRobertaForSequenceClassification(cfg)
    loaded = ours.load_weights(hf.state_dict().items())
    missing = set(dict(ours.named_parameters())) - loaded
    assert not missing, missing
    seqs = [[0, 11, 12, 13, 2], [0, 20, 21, 2, 2, 30, 31, 32, 33, 2], [0, 5, 2]]
    got = PoolingRunner(ours).run(seqs)[:, 0]
    want = []
    with torch.inference_mode():
        for s in seqs:
            want.append(hf(input_ids=torch.tensor([s])).logits[0, 0])
    want = torch.stack(want)
    assert torch.allclose(got, want, atol=1e-4), (got, want)
    # batches split by the token budget give the same scores
    got2 = PoolingRunner(ours, max_batch_tokens=8).run(seqs)[:, 0]
    assert torch.allclose(got, got2, atol=1e-5)


def test_embedding_model_is_normalised():
    cfg = RobertaConfig(vocab_size=100, hidden_size=32, num_hidden_layers=1,
                        num_attention_heads=4, intermediate_size=64, max_position_embeddings=40,
                        dtype=torch.float32)
    torch.manual_seed(1)
    m = RobertaEmbeddingModel(cfg)
    out = PoolingRunner(m).run([[0, 4, 5, 2], [0, 9, 2]])
    assert out.shape == (2, 32)
    assert torch.allclose(out.norm(dim=-1), torch.ones(2), atol=1e-5)
