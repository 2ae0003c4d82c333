"""Minimal stand-in for the two DeepSpeed names the reference's benchmark scripts import,
so that they run unmodified on a box without DeepSpeed.  Not a DeepSpeed replacement."""
