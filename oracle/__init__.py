"""CPU checkers for the attention column mean.  Test infrastructure, not product code."""
