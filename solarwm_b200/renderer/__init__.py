"""Structure-conditioned rendering on the H3-shaped DiT: observation plans, omni flow-matching core,
few-step distillation, command line."""
