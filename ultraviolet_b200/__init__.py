"""ultraviolet_b200: B200-native (sm_100a) rollout-decode path for UV-50M behind the reference's Python API."""
__version__ = "0.1.0"
