"""Tuned launch tables for the B200 kernels and the tuner that writes them."""
