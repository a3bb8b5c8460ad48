"""Operator wrappers (autograd functions) over the compiled extension."""
