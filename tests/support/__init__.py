"""Helpers shared by the tests; nothing here is shipped."""
