"""Workload descriptions for the hot path: single-op workloads that mirror the reference's
example scripts, and the nanoGPT / Llama decoder forward passes as plans."""
