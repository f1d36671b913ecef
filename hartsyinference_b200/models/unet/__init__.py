"""Convolutional U-Net denoisers (Stable Diffusion 1.5, SDXL base / refiner)."""
