"""Cross-cutting utilities: timing, logging, trackers, checkpoints, error handling."""
