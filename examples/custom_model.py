"""STAC-R on a hand-written PyTorch model: wrap two projections by name, advance the step, train.

Runs on CPU (reference arithmetic) or, when a B200 is present, on the sm_100a kernel path; nothing is downloaded.
"""

import sys
from pathlib import Path

import torch

sys.path.insert(0, str(Path(__file__).resolve().parents[1]))  # run from a checkout without installing

from stacr_b200 import apply_stacr, set_step


class TwoLayer(torch.nn.Module):
    def __init__(self, d_in=32, d_hidden=64, d_out=8):
        super().__init__()
        self.up = torch.nn.Linear(d_in, d_hidden)
        self.act = torch.nn.GELU()
        self.down = torch.nn.Linear(d_hidden, d_out)

    def forward(self, x):
        return self.down(self.act(self.up(x)))


def main(steps: int = 60) -> float:
    torch.manual_seed(42)
    device = "cuda" if torch.cuda.is_available() else "cpu"
    model = TwoLayer().to(device)
    layers = apply_stacr(model, target_names=["up", "down"], rank=8)
    optimizer = torch.optim.AdamW(model.parameters(), lr=1e-3)
    loss = None
    for step in range(steps):
        set_step(layers, step)
        optimizer.zero_grad(set_to_none=True)
        x, target = torch.randn(16, 32, device=device), torch.randn(16, 8, device=device)
        loss = (model(x) - target).square().mean()
        loss.backward()
        optimizer.step()
    print(f"loss={loss.item():.4f}; compressed projections={len(layers)}")
    return loss.item()


if __name__ == "__main__":
    main()
