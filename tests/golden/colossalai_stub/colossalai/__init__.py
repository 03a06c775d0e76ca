"""Minimal stand-in for the ColossalAI names that hpcaitech/Elixir imports, used ONLY by
tests/golden/make_golden.py to run the reference's own chunk / ElixirOptimizer code on CPU.

ColossalAI is not installable offline.  The optimizer here delegates to torch.optim.Adam / AdamW (an
implementation independent of this repository's kernels and oracle); the scaler restates
DynamicGradScaler's published update rule in Python."""
__version__ = '0.2.0'
