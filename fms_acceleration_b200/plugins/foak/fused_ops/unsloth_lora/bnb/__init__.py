"""Fused LoRA on 4-bit (NF4 / FP4) base weights."""
