"""Model assembly, the step function, the scheduler and generation."""
