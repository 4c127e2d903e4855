"""Training: trainer, optimizers, schedules, data, checkpoints, metrics."""
