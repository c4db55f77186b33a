"""Post-training: knowledge distillation and quantisation configuration."""
