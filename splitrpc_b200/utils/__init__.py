"""Configuration presets, statistics helpers and profiling utilities."""
