"""Parallel execution: process groups, fused gradient communication, launch helpers."""
from . import dist
from .dist import ensure_initialized, rank, world_size, local_rank, barrier
