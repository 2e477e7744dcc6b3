"""Small helpers shared by the execution and payload layers."""
