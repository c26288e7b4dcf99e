"""Slot-indexed call path (see :mod:`.quantized_packed_decode`)."""
