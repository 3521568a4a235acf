"""Tiny recurrent video autoencoder family (TAEHV) used as a light decoder."""
