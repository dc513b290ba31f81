"""Operator-agnostic helpers: errors, the method enum, operand validation."""
