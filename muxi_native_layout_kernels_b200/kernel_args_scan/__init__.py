"""Offline tuner that regenerates the packaged dispatch tables on the GPU it runs on."""
