"""Datasets: memory-mapped token files, GPT sample indices, samplers, blending."""
