"""Engine: model building, the step function, the scheduler and the Python entry point."""
