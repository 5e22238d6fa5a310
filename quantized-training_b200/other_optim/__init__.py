from .bf16_sr import AdamWBF16SR

__all__ = ["AdamWBF16SR"]
