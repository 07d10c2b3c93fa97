"""Kimi-K2.5 vision tower and projector."""
