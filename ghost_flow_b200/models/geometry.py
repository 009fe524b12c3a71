"""Point clouds, meshes, graph networks and reinforcement-learning agents.

* PointNet (ghostflow-nn/src/point_cloud.rs:16-529): ``PointNetConfig.default / small / large``, ``STN3d``,
  ``PointNetBackbone``, ``PointNet``, ``FarthestPointSampler``, ``KNNGrouper`` (sampling and grouping are CUDA
  kernels on GPU tensors, ``ops.render``).
* Mesh (ghostflow-nn/src/mesh.rs:17-399): ``Mesh`` (face normals, vertex adjacency, edges), ``MeshConv``,
  ``MeshPool``, ``MeshEncoder``, ``MeshUtils.create_cube / create_tetrahedron``.
* GNN (ghostflow-nn/src/gnn.rs:14-380): ``Graph``, ``GCNLayer``, ``GATLayer``, ``GraphSAGELayer`` (Mean / Max / LSTM),
  ``MPNNLayer``.
* RL (ghostflow-nn/src/rl.rs:17-534): ``ReplayBuffer``, ``QNetwork``, ``DQNAgent``, ``PolicyNetwork``,
  ``REINFORCEAgent``, ``ValueNetwork``, ``ActorCriticAgent``, ``PPOAgent.compute_gae``. The reference's train
  steps compute losses without gradients; these really update the networks.
"""
from __future__ import annotations

import enum
import random
from dataclasses import dataclass

import torch
import torch.nn.functional as F

from ..nn.layers import BatchNorm1d, Linear
from ..nn.module import Module, ModuleList, Parameter
from ..nn.rnn import LSTM
from ..ops import render


# =========================================================================== PointNet
@dataclass
class PointNetConfig:
    num_points: int = 1024
    input_dim: int = 3
    num_classes: int = 10
    use_stn: bool = True
    feature_dim: int = 1024

    @classmethod
    def default(cls): return cls()
    @classmethod
    def small(cls): return cls(512, 3, 10, False, 512)
    @classmethod
    def large(cls): return cls(2048, 3, 40, True, 2048)


class _PointMLP(Module):
    """Shared per-point MLP (a 1x1 convolution) + BatchNorm + ReLU on ``[B, N, C]``."""

    def __init__(self, cin, cout, relu=True):
        super().__init__()
        self.fc, self.bn, self.relu = Linear(cin, cout), BatchNorm1d(cout), relu

    def forward(self, x):
        B, N, _ = x.shape
        y = self.bn(self.fc(x).reshape(B * N, -1)).reshape(B, N, -1)
        return torch.relu(y) if self.relu else y


class STN3d(Module):
    """Predicts a ``k x k`` alignment transform, initialised to the identity."""

    def __init__(self, k: int = 3):
        super().__init__()
        self.k = k
        self.mlp = ModuleList([_PointMLP(k, 64), _PointMLP(64, 128), _PointMLP(128, 1024)])
        self.fc1, self.fc2, self.fc3 = Linear(1024, 512), Linear(512, 256), Linear(256, k * k)
        with torch.no_grad():
            self.fc3.weight.zero_()
            self.fc3.bias.zero_()

    def forward(self, x):
        h = x
        for m in self.mlp:
            h = m(h)
        h = h.amax(1)
        h = self.fc3(torch.relu(self.fc2(torch.relu(self.fc1(h)))))
        return h.view(-1, self.k, self.k) + torch.eye(self.k, device=x.device, dtype=x.dtype)


class PointNetBackbone(Module):
    def __init__(self, cfg: PointNetConfig):
        super().__init__()
        self.stn = STN3d(cfg.input_dim) if cfg.use_stn else None
        self.m1, self.m2 = _PointMLP(cfg.input_dim, 64), _PointMLP(64, 128)
        self.m3 = _PointMLP(128, cfg.feature_dim, relu=False)

    def forward(self, pts):
        """pts ``[B, N, 3]`` -> global feature ``[B, feature_dim]``."""
        if self.stn is not None:
            pts = torch.bmm(pts, self.stn(pts))
        return self.m3(self.m2(self.m1(pts))).amax(1)


class PointNet(Module):
    def __init__(self, config: PointNetConfig | None = None):
        super().__init__()
        self.config = c = config or PointNetConfig()
        self.backbone = PointNetBackbone(c)
        self.fc1, self.fc2, self.fc3 = Linear(c.feature_dim, 512), Linear(512, 256), Linear(256, c.num_classes)
        self.drop = torch.nn.Dropout(0.3)

    def forward(self, pts):
        h = torch.relu(self.fc1(self.backbone(pts)))
        return self.fc3(self.drop(torch.relu(self.fc2(h))))


class FarthestPointSampler:
    def __init__(self, num_samples: int):
        self.num_samples = num_samples

    def sample(self, pts, start: int = 0):
        """Indices ``[B, m]`` and the sampled points ``[B, m, 3]``."""
        idx = render.farthest_point_sample(pts, self.num_samples, start)
        return idx, torch.gather(pts, 1, idx[..., None].expand(-1, -1, pts.shape[-1]))

    __call__ = sample


class KNNGrouper:
    def __init__(self, k: int):
        self.k = k

    def group(self, pts, centers, features=None):
        """Neighbour indices ``[B, Q, k]`` and grouped (centre-relative) coordinates ``[B, Q, k, 3]``
        (+ grouped features)."""
        idx = render.knn(pts, centers, self.k)
        B, Q, K = idx.shape
        flat = idx.reshape(B, Q * K)
        g = torch.gather(pts, 1, flat[..., None].expand(-1, -1, pts.shape[-1])).view(B, Q, K, -1)
        g = g - centers[:, :, None, :]
        if features is not None:
            gf = torch.gather(features, 1, flat[..., None].expand(-1, -1, features.shape[-1])).view(B, Q, K, -1)
            return idx, g, gf
        return idx, g

    __call__ = group


# =========================================================================== meshes
class Mesh:
    def __init__(self, vertices: torch.Tensor, faces: torch.Tensor):
        self.vertices, self.faces = vertices.float(), faces.long()

    @property
    def num_vertices(self): return self.vertices.shape[0]
    @property
    def num_faces(self): return self.faces.shape[0]

    def compute_face_normals(self):
        return render.face_normals(self.vertices, self.faces)[0]

    def face_areas(self):
        return render.face_normals(self.vertices, self.faces)[1]

    def compute_vertex_normals(self):
        n, a = render.face_normals(self.vertices, self.faces)
        vn = torch.zeros_like(self.vertices)
        for k in range(3):
            vn.index_add_(0, self.faces[:, k], n * a[:, None])
        return F.normalize(vn, dim=-1)

    def edges(self):
        f = self.faces
        e = torch.cat((f[:, [0, 1]], f[:, [1, 2]], f[:, [2, 0]]), 0)
        return torch.unique(torch.sort(e, dim=1).values, dim=0)

    def vertex_adjacency(self):
        """Dense symmetric 0/1 adjacency ``[V, V]``."""
        e = self.edges()
        A = torch.zeros(self.num_vertices, self.num_vertices, device=self.vertices.device)
        A[e[:, 0], e[:, 1]] = 1
        A[e[:, 1], e[:, 0]] = 1
        return A


class MeshConv(Module):
    """Vertex feature update from itself and the mean of its neighbours."""

    def __init__(self, cin, cout):
        super().__init__()
        self.w_self, self.w_nbr = Linear(cin, cout), Linear(cin, cout, bias=False)

    def forward(self, x, adj):
        deg = adj.sum(-1, keepdim=True).clamp(min=1)
        return torch.relu(self.w_self(x) + self.w_nbr(adj @ x / deg))


class MeshPool(Module):
    """Keeps the ``ratio`` highest-scoring vertices (learned projection score)."""

    def __init__(self, channels, ratio: float = 0.5):
        super().__init__()
        self.score, self.ratio = Linear(channels, 1), ratio

    def forward(self, x, adj):
        k = max(1, int(self.ratio * x.shape[0]))
        s = self.score(x).squeeze(-1)
        idx = s.topk(k).indices
        return x[idx] * torch.sigmoid(s[idx])[:, None], adj[idx][:, idx], idx


class MeshEncoder(Module):
    def __init__(self, cin: int = 3, hidden: int = 64, out: int = 128, num_layers: int = 3):
        super().__init__()
        dims = [cin] + [hidden] * (num_layers - 1) + [out]
        self.convs = ModuleList([MeshConv(a, b) for a, b in zip(dims, dims[1:])])
        self.pools = ModuleList([MeshPool(b) for b in dims[1:-1]])

    def forward(self, mesh: Mesh):
        x, adj = mesh.vertices, mesh.vertex_adjacency()
        for i, conv in enumerate(self.convs):
            x = conv(x, adj)
            if i < len(self.pools):
                x, adj, _ = self.pools[i](x, adj)
        return x.mean(0)


class MeshUtils:
    @staticmethod
    def create_cube(size: float = 1.0) -> Mesh:
        s = size / 2
        v = torch.tensor([[-s, -s, -s], [s, -s, -s], [s, s, -s], [-s, s, -s], [-s, -s, s], [s, -s, s], [s, s, s], [-s, s, s]])
        f = torch.tensor([[0, 2, 1], [0, 3, 2], [4, 5, 6], [4, 6, 7], [0, 1, 5], [0, 5, 4], [2, 3, 7], [2, 7, 6],
                          [1, 2, 6], [1, 6, 5], [0, 4, 7], [0, 7, 3]])
        return Mesh(v, f)

    @staticmethod
    def create_tetrahedron() -> Mesh:
        v = torch.tensor([[1.0, 1, 1], [1, -1, -1], [-1, 1, -1], [-1, -1, 1]])
        f = torch.tensor([[0, 1, 2], [0, 3, 1], [0, 2, 3], [1, 3, 2]])
        return Mesh(v, f)


# =========================================================================== graph neural networks
class Graph:
    def __init__(self, num_nodes: int, edge_index: torch.Tensor, node_features: torch.Tensor | None = None,
                 edge_features: torch.Tensor | None = None):
        self.num_nodes, self.edge_index = num_nodes, edge_index.long()
        self.node_features, self.edge_features = node_features, edge_features

    def adjacency(self, self_loops: bool = False):
        A = torch.zeros(self.num_nodes, self.num_nodes, device=self.edge_index.device)
        A[self.edge_index[0], self.edge_index[1]] = 1
        if self_loops:
            A = A + torch.eye(self.num_nodes, device=A.device)
        return A

    def normalized_adjacency(self):
        A = self.adjacency(True)
        d = A.sum(1).pow(-0.5)
        return d[:, None] * A * d[None, :]


class GCNLayer(Module):
    def __init__(self, cin, cout, activation: bool = True):
        super().__init__()
        self.lin, self.activation = Linear(cin, cout), activation

    def forward(self, graph: Graph, x=None):
        x = graph.node_features if x is None else x
        h = graph.normalized_adjacency().to(x.dtype) @ self.lin(x)
        return torch.relu(h) if self.activation else h


class GATLayer(Module):
    def __init__(self, cin, cout, heads: int = 1, negative_slope: float = 0.2):
        super().__init__()
        self.heads, self.cout, self.slope = heads, cout, negative_slope
        self.lin = Linear(cin, heads * cout, bias=False)
        self.a_src = Parameter(torch.randn(heads, cout) * 0.1)
        self.a_dst = Parameter(torch.randn(heads, cout) * 0.1)

    def forward(self, graph: Graph, x=None):
        x = graph.node_features if x is None else x
        N = graph.num_nodes
        h = self.lin(x).view(N, self.heads, self.cout)
        e = F.leaky_relu((h * self.a_src).sum(-1)[:, None, :] + (h * self.a_dst).sum(-1)[None, :, :], self.slope)
        mask = graph.adjacency(True).bool()[:, :, None]
        att = torch.softmax(e.masked_fill(~mask, float("-inf")), dim=1)   # over source nodes j for target i? use [i, j]
        out = torch.einsum("ijh,jhc->ihc", att, h)
        return F.elu(out.reshape(N, self.heads * self.cout))


class SAGEAggregator(enum.Enum):
    Mean = "mean"
    Max = "max"
    Pool = "max"          # the reference's name for the max-pooling aggregator (ghostflow-nn/src/gnn.rs:224-228)
    LSTM = "lstm"


AggregatorType = SAGEAggregator


class GraphSAGELayer(Module):
    def __init__(self, cin, cout, aggregator: SAGEAggregator = SAGEAggregator.Mean):
        super().__init__()
        self.aggregator = aggregator
        self.lin = Linear(2 * cin, cout)
        self.lstm = LSTM(cin, cin, 1) if aggregator == SAGEAggregator.LSTM else None

    def forward(self, graph: Graph, x=None):
        x = graph.node_features if x is None else x
        A = graph.adjacency().to(x.dtype)
        if self.aggregator == SAGEAggregator.Mean:
            agg = A @ x / A.sum(1, keepdim=True).clamp(min=1)
        elif self.aggregator == SAGEAggregator.Max:
            agg = (x[None] + (A[:, :, None] - 1) * 1e30).amax(1)
            agg = torch.where(A.sum(1, keepdim=True) > 0, agg, torch.zeros_like(agg))
        else:
            rows = []
            for i in range(graph.num_nodes):
                nb = torch.nonzero(A[i]).flatten()
                rows.append(self.lstm(x[nb][None])[0][0, -1] if nb.numel() else torch.zeros_like(x[0]))
            agg = torch.stack(rows)
        return torch.relu(self.lin(torch.cat((x, agg), -1)))


class MPNNLayer(Module):
    """Message = MLP([h_src, h_dst, e]); update = GRU-style gate over summed messages."""

    def __init__(self, node_dim, edge_dim: int = 0, hidden: int | None = None):
        super().__init__()
        hidden = hidden or node_dim
        self.msg = torch.nn.Sequential(torch.nn.Linear(2 * node_dim + edge_dim, hidden), torch.nn.ReLU(),
                                       torch.nn.Linear(hidden, node_dim))
        self.upd = torch.nn.GRUCell(node_dim, node_dim)

    def forward(self, graph: Graph, x=None):
        x = graph.node_features if x is None else x
        src, dst = graph.edge_index
        parts = [x[src], x[dst]]
        if graph.edge_features is not None:
            parts.append(graph.edge_features)
        m = self.msg(torch.cat(parts, -1))
        agg = torch.zeros_like(x).index_add_(0, dst, m)
        return self.upd(agg, x)


# =========================================================================== reinforcement learning
@dataclass
class Experience:
    """One transition of a replay buffer (ghostflow-nn/src/rl.rs:21-28)."""
    state: torch.Tensor
    action: int
    reward: float
    next_state: torch.Tensor
    done: bool


class ReplayBuffer:
    def __init__(self, capacity: int):
        self.capacity, self.data, self.pos = capacity, [], 0

    def push(self, state, action=None, reward=None, next_state=None, done=None):
        """``push(Experience(...))`` or ``push(state, action, reward, next_state, done)``."""
        if isinstance(state, Experience):
            state, action, reward, next_state, done = (state.state, state.action, state.reward, state.next_state,
                                                       state.done)
        item = (torch.as_tensor(state, dtype=torch.float32), int(action), float(reward),
                torch.as_tensor(next_state, dtype=torch.float32), float(done))
        if len(self.data) < self.capacity:
            self.data.append(item)
        else:
            self.data[self.pos] = item
        self.pos = (self.pos + 1) % self.capacity

    def sample(self, batch_size: int, rng: random.Random | None = None):
        batch = (rng or random).sample(self.data, batch_size)
        s, a, r, s2, d = zip(*batch)
        return torch.stack(s), torch.tensor(a), torch.tensor(r), torch.stack(s2), torch.tensor(d)

    def __len__(self):
        return len(self.data)


def _mlp(i, h, o):
    return torch.nn.Sequential(torch.nn.Linear(i, h), torch.nn.ReLU(), torch.nn.Linear(h, h), torch.nn.ReLU(),
                               torch.nn.Linear(h, o))


class QNetwork(Module):
    def __init__(self, state_dim, action_dim, hidden: int = 128):
        super().__init__()
        self.net = _mlp(state_dim, hidden, action_dim)

    def forward(self, s):
        return self.net(s)


class PolicyNetwork(Module):
    def __init__(self, state_dim, action_dim, hidden: int = 128):
        super().__init__()
        self.net = _mlp(state_dim, hidden, action_dim)

    def forward(self, s):
        return torch.log_softmax(self.net(s), -1)


class ValueNetwork(Module):
    def __init__(self, state_dim, hidden: int = 128):
        super().__init__()
        self.net = _mlp(state_dim, hidden, 1)

    def forward(self, s):
        return self.net(s).squeeze(-1)


class DQNAgent:
    def __init__(self, state_dim, action_dim, lr=1e-3, gamma=0.99, epsilon=1.0, epsilon_min=0.01, epsilon_decay=0.995,
                 buffer_size=10000, batch_size=64, target_update=100):
        self.q, self.target = QNetwork(state_dim, action_dim), QNetwork(state_dim, action_dim)
        self.target.load_state_dict(self.q.state_dict())
        self.opt = torch.optim.Adam(self.q.parameters(), lr=lr)
        self.gamma, self.epsilon, self.epsilon_min, self.epsilon_decay = gamma, epsilon, epsilon_min, epsilon_decay
        self.buffer, self.batch_size, self.target_update = ReplayBuffer(buffer_size), batch_size, target_update
        self.action_dim, self.steps = action_dim, 0

    def select_action(self, state, rng: random.Random | None = None) -> int:
        if (rng or random).random() < self.epsilon:
            return (rng or random).randrange(self.action_dim)
        with torch.no_grad():
            return int(self.q(torch.as_tensor(state, dtype=torch.float32)[None]).argmax())

    def train_step(self):
        if len(self.buffer) < self.batch_size:
            return None
        s, a, r, s2, d = self.buffer.sample(self.batch_size)
        qsa = self.q(s).gather(1, a[:, None]).squeeze(1)
        with torch.no_grad():
            tgt = r + self.gamma * (1 - d) * self.target(s2).amax(1)
        loss = F.smooth_l1_loss(qsa, tgt)
        self.opt.zero_grad()
        loss.backward()
        self.opt.step()
        self.steps += 1
        self.epsilon = max(self.epsilon_min, self.epsilon * self.epsilon_decay)
        if self.steps % self.target_update == 0:
            self.target.load_state_dict(self.q.state_dict())
        return float(loss)


class REINFORCEAgent:
    def __init__(self, state_dim, action_dim, lr=1e-3, gamma=0.99):
        self.policy = PolicyNetwork(state_dim, action_dim)
        self.opt = torch.optim.Adam(self.policy.parameters(), lr=lr)
        self.gamma = gamma
        self.log_probs, self.rewards = [], []

    def select_action(self, state, generator=None) -> int:
        lp = self.policy(torch.as_tensor(state, dtype=torch.float32)[None])[0]
        a = int(torch.multinomial(lp.exp(), 1, generator=generator))
        self.log_probs.append(lp[a])
        return a

    def store_reward(self, r):
        self.rewards.append(float(r))

    def compute_returns(self):
        g, out = 0.0, []
        for r in reversed(self.rewards):
            g = r + self.gamma * g
            out.append(g)
        ret = torch.tensor(out[::-1])
        return (ret - ret.mean()) / (ret.std() + 1e-8) if ret.numel() > 1 else ret

    def update(self):
        loss = -(torch.stack(self.log_probs) * self.compute_returns()).sum()
        self.opt.zero_grad()
        loss.backward()
        self.opt.step()
        self.log_probs, self.rewards = [], []
        return float(loss)


class ActorCriticAgent:
    def __init__(self, state_dim, action_dim, lr=1e-3, gamma=0.99):
        self.actor, self.critic = PolicyNetwork(state_dim, action_dim), ValueNetwork(state_dim)
        self.opt = torch.optim.Adam(list(self.actor.parameters()) + list(self.critic.parameters()), lr=lr)
        self.gamma = gamma

    def select_action(self, state, generator=None) -> int:
        with torch.no_grad():
            lp = self.actor(torch.as_tensor(state, dtype=torch.float32)[None])[0]
        return int(torch.multinomial(lp.exp(), 1, generator=generator))

    def update(self, state, action, reward, next_state, done):
        s = torch.as_tensor(state, dtype=torch.float32)[None]
        s2 = torch.as_tensor(next_state, dtype=torch.float32)[None]
        v = self.critic(s)
        with torch.no_grad():
            tgt = reward + self.gamma * (1 - float(done)) * self.critic(s2)
        adv = (tgt - v).detach()
        loss = -(self.actor(s)[0, action] * adv).sum() + F.mse_loss(v, tgt)
        self.opt.zero_grad()
        loss.backward()
        self.opt.step()
        return float(loss)


class PPOAgent:
    def __init__(self, state_dim, action_dim, lr=3e-4, gamma=0.99, lam=0.95, clip=0.2, epochs=4):
        self.actor, self.critic = PolicyNetwork(state_dim, action_dim), ValueNetwork(state_dim)
        self.opt = torch.optim.Adam(list(self.actor.parameters()) + list(self.critic.parameters()), lr=lr)
        self.gamma, self.lam, self.clip, self.epochs = gamma, lam, clip, epochs

    def compute_gae(self, rewards, values, dones, last_value: float = 0.0):
        """Generalised advantage estimates and returns."""
        adv, g = [], 0.0
        vals = list(values) + [last_value]
        for t in reversed(range(len(rewards))):
            delta = rewards[t] + self.gamma * vals[t + 1] * (1 - dones[t]) - vals[t]
            g = delta + self.gamma * self.lam * (1 - dones[t]) * g
            adv.append(g)
        adv = torch.tensor(adv[::-1], dtype=torch.float32)
        return adv, adv + torch.tensor(list(values), dtype=torch.float32)

    def update(self, states, actions, old_log_probs, advantages, returns):
        adv = (advantages - advantages.mean()) / (advantages.std() + 1e-8)
        for _ in range(self.epochs):
            lp = self.actor(states).gather(1, actions[:, None]).squeeze(1)
            ratio = torch.exp(lp - old_log_probs)
            pol = -torch.min(ratio * adv, ratio.clamp(1 - self.clip, 1 + self.clip) * adv).mean()
            loss = pol + 0.5 * F.mse_loss(self.critic(states), returns)
            self.opt.zero_grad()
            loss.backward()
            self.opt.step()
        return float(loss)
