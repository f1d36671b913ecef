"""Diffusion schedulers and samplers."""
