"""The tensor-parallel inference engine with one rank on CPU reproduces the model zoo's greedy generation."""
import torch

from ghost_flow_b200.models.configs import LLaMAConfig
from ghost_flow_b200.models.llama import LLaMAForCausalLM
from ghost_flow_b200.parallel.tp_inference import TPLlamaInference


def test_single_rank_engine_matches_model_generate():
    cfg = LLaMAConfig(vocab_size=96, hidden_size=64, intermediate_size=128, num_hidden_layers=2,
                      num_attention_heads=4, num_key_value_heads=2, max_position_embeddings=64)
    torch.manual_seed(0)
    m = LLaMAForCausalLM(cfg, "cpu", torch.bfloat16)
    ids = torch.randint(0, 96, (2, 8))
    eng = TPLlamaInference(cfg, 2, 8, 4, "cpu", linear="nccl", weights=dict(m.state_dict()))
    assert torch.equal(eng.generate(ids, 4), m.generate(ids, 4)[:, 8:])
