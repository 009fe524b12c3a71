"""ghost_flow_b200: a Blackwell-native deep-learning framework with GhostFlow's capabilities."""
__version__ = "0.1.0"
