"""Continued-training protocols (length extension, domain adaptation) and FLOP accounting."""
