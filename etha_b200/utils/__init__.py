"""Utilities: clock sampling, profiling hooks, timing helpers."""
