# SPDX-License-Identifier: Apache-2.0
"""Compatibility helpers for code written against the reference's dependencies."""
