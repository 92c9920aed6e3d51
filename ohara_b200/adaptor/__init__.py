"""Parameter-efficient adapters: LoRA and DoRA."""
