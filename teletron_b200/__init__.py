"""teletron_b200: a Blackwell-native video-DiT training framework (Wan2.1 / HunyuanVideo flow
matching) with hand-written sm_100a kernels under a PyTorch front end."""
__version__ = "0.1.0"
