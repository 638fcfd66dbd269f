"""Multi-layer perceptron (the regression model of the asynchronous push-sum workload:
4 layers of 4096 hidden units with ReLU).  bf16 CUDA activations go through the tcgen05 GEMM."""
import torch
import torch.nn as nn

from bluefog_b200.models.gpt2 import B200Linear


class MLP(nn.Module):
    def __init__(self, in_dim=4096, hidden=4096, out_dim=1, n_layers=4, use_b200_gemm=True):
        super().__init__()
        dims = [in_dim] + [hidden] * (n_layers - 1) + [out_dim]
        self.layers = nn.ModuleList(
            [B200Linear(dims[i], dims[i + 1], use_b200_gemm=use_b200_gemm) for i in range(n_layers)])

    def forward(self, x):
        for i, layer in enumerate(self.layers):
            x = layer(x)
            if i + 1 < len(self.layers):
                x = torch.relu(x)
        return x
