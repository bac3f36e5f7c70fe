"""Heads-first wrappers with the call signatures of older releases."""
