"""siirl_b200: a Blackwell (sm_100a) native multi-controller RL post-training framework."""
__version__ = "0.1.0"
