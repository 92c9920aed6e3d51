"""Positional encodings: rotary (functional + module), ALiBi and XPos."""
