"""Offline (materialised-feature) training: dataset format, generation and replay."""
