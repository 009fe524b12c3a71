"""Worker for the tensor-parallel inference test: every linear mode against the single-GPU model."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from ghost_flow_b200.models.configs import LLaMAConfig  # noqa: E402
from ghost_flow_b200.models.llama import LLaMAForCausalLM  # noqa: E402
from ghost_flow_b200.ops import _lib  # noqa: E402
from ghost_flow_b200.parallel.tp_inference import TPLlamaInference  # noqa: E402


def main():
    out_path = sys.argv[1]
    local = int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    rank, world = dist.get_rank(), dist.get_world_size()
    cfg = LLaMAConfig(vocab_size=1024, hidden_size=512, intermediate_size=1024, num_hidden_layers=2,
                      num_attention_heads=8, num_key_value_heads=4, max_position_embeddings=512)
    torch.manual_seed(0)
    model = LLaMAForCausalLM(cfg, "cpu", torch.bfloat16)
    sd = dict(model.state_dict())
    model = model.to(dev)
    B, S, NEW = 4, 128, 6
    ids = torch.randint(0, cfg.vocab_size, (B, S), generator=torch.Generator().manual_seed(1)).to(dev)
    with torch.no_grad():
        ref_tokens = model.generate(ids, NEW)[:, S:]
        ref_logits = model(ids)[:, -1].float() if not isinstance(model(ids), tuple) else model(ids)[0][:, -1].float()
    res = {}
    for mode in ("fused", "nccl", "fp8"):
        eng = TPLlamaInference(cfg, B, S, NEW, dev, linear=mode, weights=sd)
        toks = eng.generate(ids, NEW)
        torch.cuda.synchronize()
        _lib.check_status(dev)
        # first-step logits of this rank's vocabulary slice against the reference
        eng2_logits = None
        first = eng.prefill(ids)
        lo = rank * eng.V
        sl = ref_logits[:, lo:lo + eng.V]
        res[f"{mode}_logit_rel"] = ((eng.last_logits - sl).norm() / sl.norm()).item()
        res[f"{mode}_token_agreement"] = (toks == ref_tokens).float().mean().item()
        res[f"{mode}_first_token_agreement"] = (first == ref_tokens[:, 0]).float().mean().item()
        if mode == "nccl":
            # the same decode replayed from a CUDA graph must reproduce the eager tokens exactly
            toks_g = eng.generate(ids, NEW, use_graph=True)
            torch.cuda.synchronize()
            res["graph_matches_eager"] = 0.0 if torch.equal(toks_g, toks) else 1.0
        del eng
    if rank == 0:
        torch.save(res, out_path)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
