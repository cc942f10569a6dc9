"""Reverse-mode engine and functional transforms (endia/autograd/)."""
