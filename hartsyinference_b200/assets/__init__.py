"""Model assets: checkpoint containers (safetensors, GGUF), quantisation codecs, tokenizers, chat
templates, LoRA merging, key converters and architecture detection."""
