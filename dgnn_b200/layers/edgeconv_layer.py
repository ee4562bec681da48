"""EdgeConv layer: out_i = max_j (theta(x_j - x_i) + phi(x_i)) written as
max_j (h_src[j] + h_dst[i]) with h_src = theta(x), h_dst = phi(x) - theta(x);
arguments and parameter names (theta, phi, bn) follow
dgNN/layers/edgeconv_layer.py:4-41 of the reference (whose forward, like this
one, does not apply the batch norm it creates)."""
from torch import nn

from ..operators.fused_edgeconv import EdgeConvFuse


class EdgeConv(nn.Module):
    def __init__(self, in_feat, out_feat, batch_norm=False, allow_zero_in_degree=False):
        super().__init__()
        self.batch_norm = batch_norm
        self._allow_zero_in_degree = allow_zero_in_degree
        self.theta = nn.Linear(in_feat, out_feat, bias=False)
        self.phi = nn.Linear(in_feat, out_feat, bias=False)
        if batch_norm:
            self.bn = nn.BatchNorm1d(out_feat)

    def set_allow_zero_in_degree(self, set_value):
        self._allow_zero_in_degree = set_value

    def forward(self, k, src_ind, feat):
        h_src = self.theta(feat)
        h_dst = self.phi(feat) - h_src
        return EdgeConvFuse(k, src_ind, h_src, h_dst)
