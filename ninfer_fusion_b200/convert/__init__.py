"""Offline converters: Hugging Face safetensors checkpoints <-> the engine's weight inventory / .ninfer artifacts."""
