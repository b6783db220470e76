"""neox-b200: a Blackwell-native (sm_100a) GPT-NeoX-class training framework."""
__version__ = "0.1.0"
