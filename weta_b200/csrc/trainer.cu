// Fused training-step runner.
