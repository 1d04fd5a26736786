"""Fused attention entry (``attention.cu``)."""


def supported(qkv, heads):
    return False
