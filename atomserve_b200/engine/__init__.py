"""The step function, the scheduler above it, the engine loop and its entry points."""
