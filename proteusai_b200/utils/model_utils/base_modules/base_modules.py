"""``MLP`` feed-forward block with the reference's parameter names
(``utils/model_utils/base_modules/base_modules.py:6-52``): ``in_proj``, ``hidden_proj[i]``, ``out_proj``;
activation after every layer but the last, dropout after every activation; Xavier-uniform on the first
and last layer, Kaiming-uniform on hidden layers, zero biases."""
import torch.nn as nn
import torch.nn.functional as F

from proteusai_b200.utils.model_utils.base_modules import fused_ops

_ACTS = {"gelu": F.gelu, "silu": F.silu, "relu": F.relu, "sigmoid": F.sigmoid}


class MLP(nn.Module):

    def __init__(self, d_in=512, d_out=512, d_hidden=1024, hidden_layers=0, dropout=0.1, act="gelu", zeros=False):
        super().__init__()
        self.in_proj = nn.Linear(d_in, d_hidden)
        self.hidden_proj = nn.ModuleList(nn.Linear(d_hidden, d_hidden) for _ in range(hidden_layers))
        self.out_proj = nn.Linear(d_hidden, d_out)
        self.in_dropout = nn.Dropout(dropout)
        self.hidden_dropout = nn.ModuleList(nn.Dropout(dropout) for _ in range(hidden_layers))
        self.act = _ACTS.get(act, lambda x: x)
        nn.init.xavier_uniform_(self.in_proj.weight)
        nn.init.zeros_(self.in_proj.bias)
        for layer in self.hidden_proj:
            nn.init.kaiming_uniform_(layer.weight, nonlinearity="relu")
            nn.init.zeros_(layer.bias)
        if zeros:
            nn.init.zeros_(self.out_proj.weight)
        else:
            nn.init.xavier_uniform_(self.out_proj.weight)
        nn.init.zeros_(self.out_proj.bias)

    def _act(self, x):
        # bf16 inference: the erf GELU as one HBM-bound kernel, in place on the projection's output
        if self.act is F.gelu and x.numel() % 8 == 0 and fused_ops.usable(x):
            return fused_ops.gelu(x, inplace=True)
        return self.act(x)

    def forward(self, x):
        x = self.in_dropout(self._act(self.in_proj(x)))
        for layer, drop in zip(self.hidden_proj, self.hidden_dropout):
            x = drop(self._act(layer(x)))
        return self.out_proj(x)
