"""Downstream evaluation and fine-tuning helpers."""
