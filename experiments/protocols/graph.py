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


# ------------------------------------------------------------------------------ ogbn-arxiv shaped protocol
class GraphData:
    """Node features ``x``, labels ``y`` (``[nodes, 1]``), undirected ``edge_index`` and the normalised adjacency."""

    def __init__(self, x, y, edge_index, adj):
        self.x, self.y, self.edge_index, self.adj = x, y, edge_index, adj
        self.num_nodes, self.num_edges = int(x.shape[0]), int(edge_index.shape[1])

    def to(self, device):
        return GraphData(self.x.to(device), self.y.to(device), self.edge_index.to(device), self.adj.to(device))


def _normalised_adjacency(edge_index, nodes):
    loops = torch.arange(nodes, device=edge_index.device).repeat(2, 1)
    idx = torch.cat([edge_index, edge_index.flip(0), loops], dim=1)
    adj = torch.sparse_coo_tensor(idx, torch.ones(idx.shape[1], device=edge_index.device), (nodes, nodes)).coalesce()
    adj = torch.sparse_coo_tensor(adj.indices(), torch.ones_like(adj.values()), (nodes, nodes)).coalesce()
    deg = torch.sparse.sum(adj, dim=1).to_dense().clamp_min(1)
    vals = adj.values() / torch.sqrt(deg[adj.indices()[0]] * deg[adj.indices()[1]])
    return torch.sparse_coo_tensor(adj.indices(), vals, (nodes, nodes)).coalesce()


def setup_ogbn_arxiv_data(config):
    """``(data, split_idx, info)`` for node classification on ogbn-arxiv (169 343 papers, 128 features, 40 classes).

    Loads the dataset through ``ogb`` when that package and its cache are present; otherwise builds a seeded
    homophilous graph with the same feature and class counts and ``config.graph_nodes`` nodes (default 4 000), so
    the protocol runs offline.  ``info["source"]`` says which.  Parity: experiments/protocols/graph.py:22-67.
    """
    import os
    from pathlib import Path

    seed = int(getattr(config, "seed", 0))
    try:
        from ogb.nodeproppred import NodePropPredDataset

        ds = NodePropPredDataset(name="ogbn-arxiv", root=str(Path(os.environ.get("STACR_CACHE", ".cache/stacr")) / "ogb"))
        graph, label = ds[0]
        x, y = torch.as_tensor(graph["node_feat"]).float(), torch.as_tensor(label).long().reshape(-1, 1)
        edge_index = torch.as_tensor(graph["edge_index"]).long()
        split = {k: torch.as_tensor(v).long() for k, v in ds.get_idx_split().items()}
        source = "ogbn-arxiv"
    except Exception:
        nodes = int(getattr(config, "graph_nodes", 4000))
        x, label, adj = synthetic_graph(nodes=nodes, feats=128, classes=40, avg_degree=14, seed=seed)
        idx = adj.indices()
        edge_index, y = idx[:, idx[0] < idx[1]], label.reshape(-1, 1)
        order = torch.randperm(nodes, generator=torch.Generator().manual_seed(seed))
        cut1, cut2 = int(0.54 * nodes), int(0.72 * nodes)        # the public split's proportions
        split = {"train": order[:cut1], "valid": order[cut1:cut2], "test": order[cut2:]}
        source = "synthetic"
    data = GraphData(x, y, edge_index, _normalised_adjacency(edge_index, x.shape[0]))
    info = {"num_nodes": data.num_nodes, "num_edges": data.num_edges, "num_features": int(x.shape[1]), "num_classes": int(y.max()) + 1,
            "train_size": len(split["train"]), "val_size": len(split["valid"]), "test_size": len(split["test"]), "source": source}
    return data, split, info


class GCNLayer(nn.Module):
    """``Â (x W) + b``: the linear map ``lin`` (the compression target) followed by normalised aggregation."""

    def __init__(self, fan_in, fan_out):
        super().__init__()
        self.lin = nn.Linear(fan_in, fan_out, bias=False)
        self.bias = nn.Parameter(torch.zeros(fan_out))

    def forward(self, x, adj):
        return torch.sparse.mm(adj, self.lin(x)) + self.bias


class DeepGCN(nn.Module):
    def __init__(self, in_features, hidden_features, out_features, num_layers=3, dropout=0.5):
        super().__init__()
        widths = [in_features] + [hidden_features] * (num_layers - 1) + [out_features]
        self.convs = nn.ModuleList(GCNLayer(a, b) for a, b in zip(widths[:-1], widths[1:]))
        self.bns = nn.ModuleList(nn.BatchNorm1d(hidden_features) for _ in range(num_layers - 1))
        self.dropout = dropout

    def forward(self, x, adj):
        for conv, bn in zip(self.convs[:-1], self.bns):
            x = nn.functional.dropout(torch.relu(bn(conv(x, adj))), p=self.dropout, training=self.training)
        return self.convs[-1](x, adj)


def create_gcn_model(in_features, hidden_features, out_features, num_layers=3, dropout=0.5) -> nn.Module:
    """GCN with batch norm, ReLU and dropout between layers and plain logits at the end (parity: graph.py:70-126)."""
    return DeepGCN(in_features, hidden_features, out_features, num_layers, dropout)


def get_compression_targets_gnn(model: nn.Module):
    """Names of the linear maps inside the graph convolutions (``convs.<i>.lin``)."""
    return [f"{name}.lin" for name, m in model.named_modules() if "convs" in name and isinstance(getattr(m, "lin", None), nn.Linear)]


def train_gnn_epoch(model, data, train_idx, optimizer, device=None):
    """One full-batch update; returns the loss and the training accuracy in per cent."""
    model.train()
    optimizer.zero_grad(set_to_none=True)
    out = model(data.x, data.adj)
    target = data.y[train_idx].reshape(-1)
    loss = nn.functional.cross_entropy(out[train_idx], target)
    loss.backward()
    optimizer.step()
    return {"loss": float(loss.detach()), "accuracy": 100.0 * float((out[train_idx].argmax(1) == target).float().mean())}


@torch.no_grad()
def evaluate_gnn(model, data, split_idx):
    model.eval()
    pred = model(data.x, data.adj).argmax(1)
    return {f"{k}_acc": 100.0 * float((pred[split_idx[k]] == data.y[split_idx[k]].reshape(-1)).float().mean()) for k in ("train", "valid", "test")}


def run_graph_experiment(config, logger):
    """Full-batch GCN training, dense or with STAC-R on every convolution's linear map (parity: graph.py:194-260).

    The saved activation of a wrapped layer has one row per *node*, so storage estimates use
    ``actual_batch_tokens = num_nodes``.  Runs on one device; data and tensor parallelism are rejected.
    """
    import time

    from stacr_b200.adaptive import STACRLinear as AdaptiveLinear, get_basis_pool, set_stacr_runtime_state

    from .training import estimate_storage_for_stacr, replace_linear_with_stacr

    if config.method not in ("baseline", "stacr"):
        raise ValueError("The full-batch graph protocol supports baseline or stacr")
    if getattr(config, "use_ddp", False) or getattr(config, "use_tensor_parallel", False):
        raise ValueError("The full-batch graph protocol runs on one device")
    get_basis_pool().clear()
    set_seed(int(config.seed))
    want = getattr(config, "device", "cpu")
    device = torch.device("cuda" if want in ("auto", "cuda") and torch.cuda.is_available() else "cpu")
    data, split, info = setup_ogbn_arxiv_data(config)
    model = create_gcn_model(info["num_features"], int(getattr(config, "graph_hidden", 256)), info["num_classes"], 3, 0.5)
    steps = min(int(config.epochs), int(config.max_steps or config.epochs))
    config.effective_total_steps = steps
    layers = replace_linear_with_stacr(model, get_compression_targets_gnn(model), config) if config.method == "stacr" else []
    model.to(device)
    data, split = data.to(device), {k: v.to(device) for k, v in split.items()}
    opt = torch.optim.Adam(model.parameters(), lr=float(config.lr), weight_decay=float(getattr(config, "weight_decay", 0.0)))
    if device.type == "cuda":
        torch.cuda.reset_peak_memory_stats(device)
    history, start = [], time.perf_counter()
    for step in range(steps):
        S.set_step([l for l in layers if isinstance(l, S.STACRLinear)], step)
        set_stacr_runtime_state(model, step, 0, 1, steps)
        row = train_gnn_epoch(model, data, split["train"], opt, device)
        row.update(evaluate_gnn(model, data, split))
        row["epoch"] = step + 1
        (getattr(logger, "log_metrics", None) or logger.log)(row)
        history.append(row)
    if not history:
        raise ValueError("epochs/max_steps must allow at least one graph update")
    if device.type == "cuda":
        torch.cuda.synchronize(device)
    best = max(history, key=lambda r: r["valid_acc"])
    storage = estimate_storage_for_stacr(model, config, actual_batch_tokens=info["num_nodes"]) if layers else None
    return {"status": "success", "results": {
        "epochs_completed": len(history), "best_validation_accuracy": best["valid_acc"], "test_accuracy_at_best_validation": best["test_acc"],
        "final_validation_accuracy": history[-1]["valid_acc"], "seconds": time.perf_counter() - start,
        "peak_gib": torch.cuda.max_memory_allocated(device) / 2 ** 30 if device.type == "cuda" else None,
        "wrapped_layers": sum(isinstance(m, (AdaptiveLinear, S.STACRLinear)) for m in model.modules()), "dataset": info,
        "activation_ratio": storage["achieved_ratio"] if storage else None}}


def main(argv=None) -> int:
    print(json.dumps([run("baseline"), run("stacr")], indent=2))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
