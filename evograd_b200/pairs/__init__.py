"""One candidate module per operator; see each file's docstring."""
