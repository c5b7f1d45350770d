from .seeding import seed_for, seeded_generator  # noqa: F401
