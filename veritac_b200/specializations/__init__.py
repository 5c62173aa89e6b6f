"""Specialization packages of the B200 back end; implementations are loaded explicitly."""
