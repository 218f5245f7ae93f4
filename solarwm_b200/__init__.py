"""solarwm_b200: a Blackwell-native (sm_100a) framework for camera-controlled video world models."""
__version__ = "0.1.0"
