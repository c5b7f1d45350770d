"""Evaluation harness: launcher, per-rank worker, output compare, timing, roofline, reports."""
