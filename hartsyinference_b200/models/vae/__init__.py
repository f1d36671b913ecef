"""VAE decoders: 2-D (Flux / SD families) and causal 3-D (Wan)."""
