"""Evaluation helpers for rendered videos: ground-truth metrics, edge adherence, pairwise ratings."""
