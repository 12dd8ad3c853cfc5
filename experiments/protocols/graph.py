"""Graph-network protocol: a two-layer GCN on a synthetic citation-style graph with STAC-R on its linear maps.

The reference runs this on ogbn-arxiv through PyTorch Geometric and reports it as a *negative* result (GNN
activations after sparse aggregation are not low-rank enough for rank-8 tracking to pay).  This version needs no
external graph library: aggregation is a normalised sparse adjacency product, and the graph is a seeded
stochastic-block-model so it runs offline.  Parity: experiments/protocols/graph.py of the reference project.
"""

from __future__ import annotations

import json

import torch
from torch import nn

import stacr_b200 as S
from stacr_b200.utils import set_seed


def synthetic_graph(nodes=2000, feats=128, classes=8, avg_degree=12, seed=0):
    gen = torch.Generator().manual_seed(seed)
    label = torch.randint(0, classes, (nodes,), generator=gen)
    centers = torch.randn(classes, feats, generator=gen)
    x = centers[label] + 1.5 * torch.randn(nodes, feats, generator=gen)
    n_edges = nodes * avg_degree // 2
    src = torch.randint(0, nodes, (n_edges,), generator=gen)
    same = torch.rand(n_edges, generator=gen) < 0.7
    dst = torch.randint(0, nodes, (n_edges,), generator=gen)
    # rewire 70 % of edges to a node of the same class (homophily)
    perm = torch.argsort(label + torch.rand(nodes, generator=gen) * 0.5)
    rank_of = torch.empty_like(perm)
    rank_of[perm] = torch.arange(nodes)
    neighbour = perm[(rank_of[src] + torch.randint(1, 20, (n_edges,), generator=gen)).clamp_max(nodes - 1)]
    dst = torch.where(same, neighbour, dst)
    idx = torch.cat([torch.stack([src, dst]), torch.stack([dst, src]), torch.arange(nodes).repeat(2, 1)], dim=1)
    adj = torch.sparse_coo_tensor(idx, torch.ones(idx.shape[1]), (nodes, nodes)).coalesce()
    deg = torch.sparse.sum(adj, dim=1).to_dense().clamp_min(1)
    vals = adj.values() / torch.sqrt(deg[adj.indices()[0]] * deg[adj.indices()[1]])
    return x, label, torch.sparse_coo_tensor(adj.indices(), vals, (nodes, nodes)).coalesce()


class GCN(nn.Module):
    def __init__(self, feats, hidden, classes):
        super().__init__()
        self.lin1, self.lin2 = nn.Linear(feats, hidden), nn.Linear(hidden, classes)

    def forward(self, x, adj):
        h = torch.relu(torch.sparse.mm(adj, self.lin1(x)))
        return torch.sparse.mm(adj, self.lin2(h))


def run(method="stacr", epochs=30, hidden=256, seed=42, rank=8, budget=0.005) -> dict:
    set_seed(seed)
    x, y, adj = synthetic_graph(seed=seed)
    model = GCN(x.shape[1], hidden, int(y.max()) + 1)
    layers = S.apply_stacr(model, surface="all", min_features=1, rank=rank, residual_budget=budget, turbo_after_step=None) if method == "stacr" else []
    opt = torch.optim.Adam(model.parameters(), lr=1e-2)
    train = torch.arange(x.shape[0]) % 5 != 0
    for epoch in range(epochs):
        S.set_step(layers, epoch)
        opt.zero_grad()
        loss = nn.functional.cross_entropy(model(x, adj)[train], y[train])
        loss.backward()
        opt.step()
    model.eval()
    with torch.no_grad():
        acc = float((model(x, adj)[~train].argmax(-1) == y[~train]).float().mean())
    return {"method": method, "test_accuracy": acc, "final_loss": float(loss.detach()), "wrapped": len(layers)}


def main(argv=None) -> int:
    print(json.dumps([run("baseline"), run("stacr")], indent=2))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
