"""Drop-in replacements for the attention building blocks of ``pithtrain.operators``."""
