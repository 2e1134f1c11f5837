"""Architecture modules: each turns its configuration into a plan and registers itself."""
