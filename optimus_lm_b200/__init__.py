"""B200-native MoE pretraining framework with the capabilities of IntelLabs/Optimus-LM."""
__version__ = "0.1.0"
