"""Agentic (multi-turn, tool-using, asynchronous) reinforcement learning."""
