"""Example models that exercise the gw8 layer through ``spio_b200.transform``."""
