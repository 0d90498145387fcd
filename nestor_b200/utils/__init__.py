"""Process-group helpers, logging, seeding, timing."""
