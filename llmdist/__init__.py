"""Distributed wrappers; thin aliases of ``systems_for_llms_b200.parallel``."""
