"""Shared parameter-version counter (importable without the native library)."""
EPOCH = [0]
