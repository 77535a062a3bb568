"""Operators: each op has a hand-written sm_100a CUDA implementation and a torch reference."""
