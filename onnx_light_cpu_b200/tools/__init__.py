"""Measurement and parity tools (CUDA counterparts of the reference's tools/ directory)."""
