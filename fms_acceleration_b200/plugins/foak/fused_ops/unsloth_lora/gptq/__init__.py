"""Fused LoRA on GPTQ base weights."""
