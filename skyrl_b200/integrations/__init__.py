"""Integrations: trainers that keep the RL loop of this package but hand the GPU work to another system."""
