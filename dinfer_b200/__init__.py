"""dinfer_b200: a small, whole inference engine for one B200 (sm_100a), from a model folder
(config.json + safetensors) to generated tokens."""
__version__ = "0.1.0"
