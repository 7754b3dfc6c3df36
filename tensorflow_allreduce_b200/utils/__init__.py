"""Helpers around the library: statistics/timeline, clock sampling, multi-process test spawning."""
