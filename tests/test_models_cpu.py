"""Model zoo on CPU: shapes, a few closed-form checks, and that tiny models train."""
import math

import torch
import torch.nn.functional as F

from ghost_flow_b200 import models as M
from ghost_flow_b200.ops import render


def test_llama_tiny_trains_and_generates_with_cache():
    torch.manual_seed(0)
    cfg = M.LLaMAConfig.llama_tiny()
    m = M.LLaMAForCausalLM(cfg)
    ids = torch.randint(0, cfg.vocab_size, (2, 17))
    opt = torch.optim.AdamW(m.parameters(), lr=3e-3)
    first = None
    for _ in range(8):
        loss, _ = m(ids[:, :-1], labels=ids[:, 1:])
        opt.zero_grad(); loss.backward(); opt.step()
        first = first or loss.item()
    assert loss.item() < first
    m.eval()
    out = m.generate(ids[:, :5], 4)
    assert out.shape == (2, 9)
    # cached decoding equals a full forward
    full = m(out[:, :-1])[:, -1].argmax(-1)
    assert torch.equal(full, out[:, -1])


def test_engine_and_module_agree():
    from ghost_flow_b200.parallel.zero3 import Zero3LlamaEngine
    cfg = M.LLaMAConfig.llama_tiny()
    eng = Zero3LlamaEngine(cfg, "cpu", dtype=torch.float32, seed=1)
    m = M.LLaMAForCausalLM(cfg)
    m.load_engine_state(eng.state_dict())
    ids = torch.randint(0, cfg.vocab_size, (2, 16))
    assert torch.allclose(eng.forward_logits(ids), m(ids), atol=1e-4)


def test_gpt_bert_vit_t5_mixtral_shapes():
    g = M.GPTForCausalLM(M.GPTConfig.gpt_tiny()); g.eval()
    ids = torch.randint(0, 1000, (2, 12))
    assert g(ids).shape == (2, 12, 1000)
    gen = g.generate(ids[:, :4], 3)
    assert gen.shape == (2, 7) and torch.equal(g(gen[:, :-1])[:, -1].argmax(-1), gen[:, -1])
    b = M.BertModel(M.BertConfig.bert_tiny()); b.eval()
    out = b(ids, attention_mask=torch.ones(2, 12))
    assert out.last_hidden_state.shape == (2, 12, 128) and out.pooler_output.shape == (2, 128)
    # the attention mask matters: masking the tail changes the head's representation
    mask = torch.ones(2, 12); mask[:, 6:] = 0
    assert not torch.allclose(b(ids, attention_mask=mask).last_hidden_state[:, 0], out.last_hidden_state[:, 0])
    assert M.BertForSequenceClassification(M.BertConfig.bert_tiny(), 3)(ids).shape == (2, 3)
    v = M.VisionTransformer(M.ViTConfig.vit_tiny())
    assert v(torch.randn(2, 3, 32, 32)).shape == (2, 10)
    t5 = M.T5ForConditionalGeneration(M.T5Config.t5_tiny()); t5.eval()
    loss, logits = t5(ids, ids[:, :5], labels=ids[:, 1:6])
    assert logits.shape == (2, 5, 1000) and loss.item() > 0 and t5.generate(ids, 3).shape[1] <= 4
    mx = M.MixtralForCausalLM(M.MixtralConfig.mixtral_tiny())
    loss, _ = mx(ids[:, :-1], labels=ids[:, 1:])
    loss.backward()
    assert mx.layers[0].moe.router.gate.weight.grad is not None and float(mx.aux_loss()) > 0


def test_clip_diffusion():
    c = M.CLIP(M.CLIPConfig.tiny())
    li, lt = c(torch.randn(3, 3, 32, 32), torch.randint(0, 100, (3, 16)))
    assert li.shape == (3, 3) and torch.allclose(li, lt.t())
    assert abs(c.logit_scale.item() - math.log(1 / 0.07)) < 1e-3
    s = M.NoiseScheduler(M.DiffusionConfig.tiny())
    x0, n = torch.randn(2, 3, 8, 8), torch.randn(2, 3, 8, 8)
    t = torch.tensor([3, 50])
    assert torch.allclose(s.predict_x0(s.add_noise(x0, n, t), n, t), x0, atol=1e-4)
    d = M.DDPM(M.DiffusionConfig.tiny())
    assert d(torch.randn(2, 3, 32, 32)).item() > 0
    assert d.sample((1, 3, 32, 32), num_steps=2).shape == (1, 3, 32, 32)


def test_nerf_volume_rendering_closed_form():
    # a fully opaque red slab at the first sample renders pure red at that depth
    rgb = torch.zeros(1, 4, 3); rgb[0, 0] = torch.tensor([1.0, 0, 0])
    sigma = torch.tensor([[1e4, 0, 0, 0]]); z = torch.tensor([[2.0, 3.0, 4.0, 5.0]])
    color, depth, acc, w = render.volume_render(rgb, sigma, z)
    assert torch.allclose(color, torch.tensor([[1.0, 0, 0]]), atol=1e-4) and abs(depth.item() - 2.0) < 1e-3
    assert abs(acc.item() - 1) < 1e-4
    pe = render.positional_encoding(torch.tensor([[0.5, 1.0]]), 2)
    assert pe.shape == (1, 10) and abs(pe[0, 1].item() - math.sin(0.5)) < 1e-6 and abs(pe[0, 4].item() - math.cos(1.0)) < 1e-6
    out = M.NeRF(M.NeRFConfig.tiny()).render(torch.zeros(5, 3), F.normalize(torch.randn(5, 3), dim=-1))
    assert out["color"].shape == (5, 3) and out["depth"].shape == (5,)


def test_pointcloud_mesh_gnn_rl():
    pts = torch.randn(2, 64, 3)
    idx, sub = M.FarthestPointSampler(8)(pts)
    assert idx.shape == (2, 8) and len(set(idx[0].tolist())) == 8
    nn_idx, grouped = M.KNNGrouper(4)(pts, sub)
    assert nn_idx.shape == (2, 8, 4) and torch.equal(nn_idx[:, :, 0], idx)     # nearest neighbour of a sample is itself
    assert M.PointNet(M.PointNetConfig(64, 3, 5, True, 128))(pts).shape == (2, 5)
    cube = M.MeshUtils.create_cube()
    n = cube.compute_face_normals()
    assert torch.allclose(n.norm(dim=-1), torch.ones(12)) and abs(cube.face_areas().sum().item() - 6.0) < 1e-5
    assert cube.edges().shape[0] == 18 and M.MeshEncoder(3, 8, 16)(cube).shape == (16,)
    g = M.Graph(4, torch.tensor([[0, 1, 2, 3, 1], [1, 0, 3, 2, 2]]), torch.randn(4, 6))
    for layer in (M.GCNLayer(6, 5), M.GATLayer(6, 5, 2), M.GraphSAGELayer(6, 5), M.GraphSAGELayer(6, 5, M.SAGEAggregator.Max),
                  M.GraphSAGELayer(6, 5, M.SAGEAggregator.LSTM)):
        assert layer(g).shape[0] == 4
    assert M.MPNNLayer(6)(g).shape == (4, 6)
    agent = M.DQNAgent(4, 2, batch_size=8)
    for i in range(16):
        agent.buffer.push(torch.randn(4), i % 2, 1.0, torch.randn(4), False)
    assert agent.train_step() is not None
    adv, ret = M.PPOAgent(4, 2).compute_gae([1.0, 1.0], [0.5, 0.5], [0, 1])
    assert abs(adv[1].item() - 0.5) < 1e-6 and abs(ret[1].item() - 1.0) < 1e-6
