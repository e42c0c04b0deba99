"""Quantisation codecs: E8P lattice (Q4 two-stage, Q2), W8, A8 and INT8 KV."""
from . import e8p  # noqa: F401
