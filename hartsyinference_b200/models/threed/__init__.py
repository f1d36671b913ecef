"""Single-image 3-D reconstruction models."""
