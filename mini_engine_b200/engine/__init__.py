"""Sequences, the scheduler, the step function, the engine loop and trace replay."""
