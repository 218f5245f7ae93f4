"""Realtime serving: block-causal streaming generation, camera control, frame sink, HTTP front end."""
