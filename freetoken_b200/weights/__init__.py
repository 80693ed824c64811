"""Weights: safetensors reading and writing, binding by name, seeded random weights."""
