"""The engine: step function, scheduler, trace replay, command line."""
