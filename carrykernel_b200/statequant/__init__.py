"""statequant operator surface (see :mod:`.kernel`)."""
