"""Helpers shipped with the framework (testing utilities)."""
