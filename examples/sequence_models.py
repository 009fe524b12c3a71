"""LSTM / GRU / bidirectional LSTM and a Transformer encoder on a [8, 128, 512] batch
(the shapes of the reference's examples/sequence_models.rs)."""
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from ghost_flow_b200 import nn  # noqa: E402


def main():
    dev = "cuda" if torch.cuda.is_available() else "cpu"
    x = torch.randn(8, 32, 50, device=dev)
    lstm = nn.LSTM(50, 128, 2, False, 0.1).to(dev)
    out, _ = lstm(x)
    print("LSTM", tuple(out.shape))
    gru = nn.GRU(50, 128, 1, False, 0.0).to(dev)
    out, _ = gru(x)
    print("GRU", tuple(out.shape))
    bi = nn.LSTM(50, 64, 1, True, 0.0).to(dev)
    out, _ = bi(x)
    print("BiLSTM", tuple(out.shape))
    enc = nn.TransformerEncoder(512, 8, 2048, 2, 0.1).to(dev).eval()
    seq = torch.randn(8, 128, 512, device=dev)
    with torch.no_grad():
        print("TransformerEncoder", tuple(enc(seq).shape))


if __name__ == "__main__":
    main()
