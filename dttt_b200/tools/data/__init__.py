"""Data acquisition and decontamination tools (host-side; no GPU)."""
