"""Offline tools: result extraction, plotting, consensus step-size tuning."""
