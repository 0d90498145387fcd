"""Training loop, optimizer, losses, checkpointing and memory levers."""
