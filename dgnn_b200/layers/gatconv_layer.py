"""GATConv layer: dense projection on the tensor cores (operators/projection.py), attention
logits and the sparse softmax-aggregation through the fused operators.  Constructor arguments,
parameter names (W, attn_l, attn_r, bias, res_fc), initialisation and forward
signature follow dgNN/layers/gatconv_layer.py:7-92 of the reference, so
state_dicts interchange."""
import math

import torch
from torch import nn

from .. import kernels
from ..operators.fused_gatconv import GATConvFuse, GATConvFuse_inference, GATLayerFuse
from ..operators.projection import project


class GATConv(nn.Module):
    def __init__(self, in_feats, out_feats, num_heads, feat_drop=0., attn_drop=0., negative_slope=0.2,
                 residual=False, activation=None, bias=True):
        super().__init__()
        self.in_feats, self.out_feats, self.num_heads = in_feats, out_feats, num_heads
        self.negative_slope = negative_slope
        self.attn_drop = attn_drop
        self.activation = activation
        hf = num_heads * out_feats
        self.W = nn.Parameter(torch.empty(in_feats, hf))
        self.attn_l = nn.Parameter(torch.empty(1, num_heads, out_feats))
        self.attn_r = nn.Parameter(torch.empty(1, num_heads, out_feats))
        self.feat_drop = nn.Dropout(feat_drop)
        if bias:
            self.bias = nn.Parameter(torch.empty(hf))
        else:
            self.register_buffer("bias", None)
        if residual:
            self.res_fc = nn.Linear(in_feats, hf, bias=False) if in_feats != hf else nn.Identity()
        else:
            self.register_buffer("res_fc", None)
        self.reset_parameters()

    def reset_parameters(self):
        """Xavier-normal with the ReLU gain for W, attn_l, attn_r (and res_fc), zero bias
        (gatconv_layer.py:46-66 of the reference)."""
        gain = math.sqrt(2.0)
        for p in (self.W, self.attn_l, self.attn_r):
            nn.init.xavier_normal_(p, gain=gain)
        if self.bias is not None:
            nn.init.zeros_(self.bias)
        if isinstance(self.res_fc, nn.Linear):
            nn.init.xavier_normal_(self.res_fc.weight, gain=gain)

    def forward(self, row_ptr, col_ind, col_ptr, row_ind, permute, feat):
        heads, width = self.num_heads, self.out_feats
        h = self.feat_drop(project(feat, self.W).view(-1, heads, width))
        # destination (row) logits use attn_l, source (column) logits use attn_r
        fused_logits = h.is_cuda and kernels.logits_supported(heads, width)
        if self.training and fused_logits:
            # logits, aggregation and their backward as one autograd node (same math as the branch below)
            # without a residual branch the bias is added in the aggregation kernel's epilogue
            fuse_bias = self.bias is not None and self.res_fc is None
            rst = GATLayerFuse(h, self.attn_l, self.attn_r, row_ptr, col_ind, col_ptr, row_ind, permute,
                               self.negative_slope, self.attn_drop, self.bias if fuse_bias else None)
            if fuse_bias:
                return self.activation(rst) if self.activation else rst
        else:
            if fused_logits and not torch.is_grad_enabled():
                attn_row, attn_col = kernels.gat_logits_forward(h, self.attn_l, self.attn_r)
            else:
                attn_row = (h * self.attn_l).sum(-1)
                attn_col = (h * self.attn_r).sum(-1)
            if self.training:
                rst = GATConvFuse(attn_row, attn_col, row_ptr, col_ind, col_ptr, row_ind, permute,
                                  self.negative_slope, h, self.attn_drop)
            else:
                rst = GATConvFuse_inference(attn_row, attn_col, row_ptr, col_ind, self.negative_slope, h)
        if self.res_fc is not None:
            # as in the reference the residual branch is applied to the projected features
            rst = rst + self.res_fc(h).view(-1, heads, width)
        if self.bias is not None:
            rst = rst + self.bias.view(-1, heads, width)
        return self.activation(rst) if self.activation else rst
