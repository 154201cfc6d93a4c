"""Command-line tools: launcher, preflight, init-latency sweep, size sweep, tuning, plots."""
