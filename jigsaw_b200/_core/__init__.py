"""Runtime internals shared by every layer (communication, autocast, buffers, placement)."""
