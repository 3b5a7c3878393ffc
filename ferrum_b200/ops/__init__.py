"""Kernel launchers and autograd-aware ops."""
