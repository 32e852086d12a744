"""Helpers that touch the outside world (model hubs, object stores)."""
