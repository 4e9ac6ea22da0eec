"""Step function, scheduler and the Python entry point."""
