"""Single-device training stack; thin aliases of ``systems_for_llms_b200``."""
