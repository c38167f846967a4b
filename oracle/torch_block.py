"""CPU baseline for the benchmark: the GPT-2 style block, the MLP and the fused ops in eager
PyTorch float32 (oneDNN) on the host cores.

TEST / BENCHMARK INFRASTRUCTURE ONLY -- never imported by the package.  The reference's own CPU
implementation of this path is its MLIR backend (kiln/codegen, kiln/runtime), which needs LLVM's
Python bindings and cannot be built offline; its README places that pipeline within 5 % of eager
PyTorch at one thread (README.md:88-91), so eager PyTorch on the same tensors stands in for it.
The arithmetic restates the model of the reference's tests (tests/models/transformer.py:14-28:
pre-LN, fused QKV projection, causal additive mask, softmax scaled by 1/sqrt(head dim), tanh-GELU
MLP, two residual adds) functionally, from module-style parameter dictionaries.
"""

from __future__ import annotations

import math

import torch
import torch.nn.functional as F


def to_torch(params, dtype=torch.float32):
    return {k: torch.from_numpy(v).to(dtype) for k, v in params.items()}


def block_forward(p, x, heads=12, eps=1e-5):
    """x: [T, C]. p: ln1/ln2/c_attn/c_proj/fc/proj weights and biases, 'mask' [T, T]."""
    t, c = x.shape
    hd = c // heads
    h = F.layer_norm(x, (c,), p["ln1.weight"], p["ln1.bias"], eps)
    qkv = F.linear(h, p["c_attn.weight"], p["c_attn.bias"])
    q, k, v = (z.reshape(t, heads, hd).transpose(0, 1) for z in qkv.split(c, dim=1))
    att = torch.softmax(q @ k.transpose(-2, -1) * (1.0 / math.sqrt(hd)) + p["mask"], dim=-1)
    y = (att @ v).transpose(0, 1).reshape(t, c)
    x = x + F.linear(y, p["c_proj.weight"], p["c_proj.bias"])
    h = F.layer_norm(x, (c,), p["ln2.weight"], p["ln2.bias"], eps)
    return x + F.linear(F.gelu(F.linear(h, p["fc.weight"], p["fc.bias"]), approximate="tanh"),
                        p["proj.weight"], p["proj.bias"])


def mlp_forward(p, x):
    return F.linear(F.gelu(F.linear(x, p["0.weight"], p["0.bias"]), approximate="tanh"), p["2.weight"], p["2.bias"])
