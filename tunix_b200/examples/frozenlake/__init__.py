"""Multi-turn grid-world environment for agentic RL (the reference ships the same game under
examples/frozenlake)."""
from .env import FrozenLakeEnv, FrozenLakeAgent, generate_map
