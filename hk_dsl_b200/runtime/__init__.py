"""The C-ABI library's loader and the torch custom-op surface built on it."""
