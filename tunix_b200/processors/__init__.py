"""Host-side preprocessing of images and audio for multimodal decoders."""
