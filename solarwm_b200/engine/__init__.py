"""Model-independent engines: training state machine, objectives, optimizer, inference."""
