"""Authentication and administration routes (crates/axonml-server/src/api/auth.rs; route table
api/mod.rs:111-146, 342-350): register (with e-mail verification when a mail service is
configured), login (with the MFA hand-off token), logout, refresh, me, TOTP setup / enable /
verify, WebAuthn registration and assertion, recovery codes, MFA disable, user administration,
admin query."""
from __future__ import annotations

import hashlib
import os
import time

from . import auth as A
from . import webauthn as W
from .api import ADMIN, PUBLIC, USER, HttpError
from .store import now_iso


def register(app) -> None:
    r = app.router

    def _login_response(u: dict, mfa_verified: bool) -> dict:
        app.users.update(u["id"], {"last_login": now_iso()})
        pair = app.jwt.create_token_pair(u["id"], u["email"], u["role"], mfa_verified)
        return {**pair, "user": app.public_user(u), "requires_mfa": False}

    def auth_register(req):
        # allow_registration: True = anyone may register, False = nobody, None (default) = only the
        # first account, which becomes the administrator and creates the others.
        if app.allow_registration is False or (app.allow_registration is None and app.users.count() > 0):
            raise HttpError(403, "registration is disabled; ask an administrator for an account")
        email, name, password = req.need("email", "name", "password")
        if "@" not in email or len(password) < 8:
            raise HttpError(400, "a valid e-mail address and a password of at least 8 characters are required")
        role = "admin" if app.users.count() == 0 else "user"      # the first account administers the server
        u = app.create_user(email, name, password, role)
        if role == "user" and app.email.is_configured():
            # the address has to be confirmed through the mailed link before the account can sign in
            token = os.urandom(24).hex()
            u = app.users.update(u["id"], {"email_verified": False, "approved": False,
                                           "verify_token_hash": hashlib.sha256(token.encode()).hexdigest(),
                                           "verify_expires": time.time() + 24 * 3600})
            try:
                app.email.send_verification_email(u["email"], u["name"], f"{app.public_url}/api/auth/verify-email?token={token}")
                for adm in app.users.find({"role": "admin"}):
                    app.email.send_admin_signup_notification(adm["email"], u["email"], u["name"])
            except Exception as e:                      # the account exists; an administrator can still approve it
                return 201, {"user": app.public_user(u), "message": f"registered; the verification e-mail could not be sent ({e})"}
            return 201, {"user": app.public_user(u), "message": "registered; check your inbox for the verification link"}
        return 201, {"user": app.public_user(u), "message": "registered"}

    def auth_verify_email(req):
        token = req.q("token") or (req.json or {}).get("token")
        if not token:
            raise HttpError(400, "token is required")
        u = app.users.find_one(verify_token_hash=hashlib.sha256(str(token).encode()).hexdigest())
        if u is None or time.time() > float(u.get("verify_expires") or 0):
            raise HttpError(400, "the verification link is invalid or has expired")
        u = app.users.update(u["id"], {"email_verified": True, "approved": True, "verify_token_hash": None,
                                       "verify_expires": None})
        try:
            app.email.send_welcome_email(u["email"], u["name"], app.public_url)
        except Exception:
            pass
        return {"user": app.public_user(u), "message": "e-mail address verified"}

    def auth_login(req):
        email, password = req.need("email", "password")
        u = app.users.find_one(email=email.lower())
        if u is None or not A.verify_password(password, u["password_hash"]):
            raise HttpError(401, "invalid e-mail or password")
        if not u.get("email_verified", True):
            raise HttpError(403, "e-mail address not verified yet")
        if not u.get("approved", True):
            raise HttpError(403, "account not approved yet")
        if u.get("mfa_enabled") or u.get("webauthn_credentials"):
            methods = (["totp", "recovery"] if u.get("mfa_enabled") else []) + (["webauthn"] if u.get("webauthn_credentials") else [])
            return {"requires_mfa": True, "mfa_methods": methods, **app.jwt.create_mfa_token(u["id"], u["email"])}
        return _login_response(u, False)

    def _mfa_user(req) -> dict:
        (tok,) = req.need("mfa_token")
        c = app.jwt.validate_mfa_token(tok)
        return app.users.get(c.sub)

    def mfa_totp_verify(req):
        u = _mfa_user(req)
        (code,) = req.need("code")
        if not u.get("totp_secret") or not app.totp.verify(u["totp_secret"], str(code)):
            raise HttpError(401, "invalid code")
        return _login_response(u, True)

    def mfa_recovery_use(req):
        u = _mfa_user(req)
        (code,) = req.need("code")
        i = A.RecoveryAuth.verify_code(str(code), u.get("recovery_codes") or [])
        if i is None:
            raise HttpError(401, "invalid recovery code")
        left = list(u["recovery_codes"])
        del left[i]                                  # a recovery code works once
        app.users.update(u["id"], {"recovery_codes": left})
        out = _login_response(u, True)
        out["recovery_codes_left"] = len(left)
        return out

    def auth_logout(req):
        tok = A.JwtAuth.extract_from_header(req.headers.get("Authorization"))
        if tok:
            app.revoked.add(tok)
        return {"message": "logged out"}

    def auth_refresh(req):
        (tok,) = req.need("refresh_token")
        c = app.jwt.validate_refresh_token(tok)
        u = app.users.get(c.sub)                     # a deleted user cannot refresh
        return app.jwt.create_token_pair(u["id"], u["email"], u["role"])

    def auth_me(req):
        return app.public_user(app.users.get(req.user_id))

    def totp_setup(req):
        u = app.users.get(req.user_id)
        s = app.totp.setup(u["email"])
        app.users.update(u["id"], {"pending_totp_secret": s["secret"]})
        return s

    def totp_enable(req):
        u = app.users.get(req.user_id)
        (code,) = req.need("code")
        secret = u.get("pending_totp_secret")
        if not secret or not app.totp.verify(secret, str(code)):
            raise HttpError(400, "code does not match the pending secret")
        rc = A.RecoveryAuth.generate_codes(10)
        app.users.update(u["id"], {"totp_secret": secret, "pending_totp_secret": None, "mfa_enabled": True,
                                   "recovery_codes": rc["hashed_codes"]})
        return {"mfa_enabled": True, "recovery_codes": rc["codes"]}

    def recovery_generate(req):
        rc = A.RecoveryAuth.generate_codes(10)
        app.users.update(req.user_id, {"recovery_codes": rc["hashed_codes"]})
        return {"recovery_codes": rc["codes"]}

    def recovery_status(req):
        return {"remaining": len(app.users.get(req.user_id).get("recovery_codes") or [])}

    def mfa_disable(req):
        u = app.users.get(req.user_id)
        (password,) = req.need("password")
        if not A.verify_password(password, u["password_hash"]):
            raise HttpError(401, "wrong password")
        app.users.update(u["id"], {"mfa_enabled": False, "totp_secret": None, "pending_totp_secret": None,
                                   "recovery_codes": [], "webauthn_credentials": []})
        return {"mfa_enabled": False}

    # ------------------------------------------------------------------ WebAuthn
    def _webauthn():
        if not W.available():
            raise HttpError(501, "WebAuthn needs the 'cryptography' package on the server; use TOTP")
        return app.webauthn

    def _webauthn_call(fn, *args):
        try:
            return fn(*args)
        except W.WebAuthnError as e:
            raise HttpError(400, str(e)) from None

    def webauthn_register_start(req):
        u = app.users.get(req.user_id)
        return _webauthn_call(_webauthn().start_registration, u["id"], u["email"], u["name"], u.get("webauthn_credentials") or [])

    def webauthn_register_finish(req):
        u = app.users.get(req.user_id)
        body = req.json or {}
        cred = _webauthn_call(_webauthn().finish_registration, u["id"], body.get("credential") or body, str(body.get("name") or ""))
        creds = list(u.get("webauthn_credentials") or [])
        if any(c["credential_id"] == cred["credential_id"] for c in creds):
            raise HttpError(409, "this credential is already registered")
        creds.append(cred)
        app.users.update(u["id"], {"webauthn_credentials": creds})
        return 201, {"credential": {k: cred[k] for k in ("credential_id", "name", "created_at")}, "webauthn_enabled": True}

    def webauthn_auth_start(req):
        u = _mfa_user(req)
        return _webauthn_call(_webauthn().start_authentication, u["id"], u.get("webauthn_credentials") or [])

    def webauthn_auth_finish(req):
        u = _mfa_user(req)
        body = req.json or {}
        creds = list(u.get("webauthn_credentials") or [])
        used = _webauthn_call(_webauthn().finish_authentication, u["id"], body.get("credential") or body, creds)
        creds = [used if c["credential_id"] == used["credential_id"] else c for c in creds]
        app.users.update(u["id"], {"webauthn_credentials": creds})
        return _login_response(u, True)

    def webauthn_list(req):
        u = app.users.get(req.user_id)
        return [{k: c.get(k) for k in ("credential_id", "name", "created_at", "counter")} for c in u.get("webauthn_credentials") or []]

    def webauthn_delete(req):
        u = app.users.get(req.user_id)
        left = [c for c in u.get("webauthn_credentials") or [] if c["credential_id"] != req.params["cred"]]
        if len(left) == len(u.get("webauthn_credentials") or []):
            raise HttpError(404, "no such credential")
        app.users.update(u["id"], {"webauthn_credentials": left})
        return {"deleted": True, "webauthn_enabled": bool(left)}

    r.add("POST", "/api/auth/register", auth_register, PUBLIC)
    r.add("POST", "/api/auth/login", auth_login, PUBLIC)
    r.add("POST", "/api/auth/mfa/totp/verify", mfa_totp_verify, PUBLIC)
    r.add("POST", "/api/auth/mfa/recovery", mfa_recovery_use, PUBLIC)
    r.add("GET", "/api/auth/verify-email", auth_verify_email, PUBLIC)
    r.add("POST", "/api/auth/verify-email", auth_verify_email, PUBLIC)
    r.add("POST", "/api/auth/mfa/webauthn/authenticate/start", webauthn_auth_start, PUBLIC)
    r.add("POST", "/api/auth/mfa/webauthn/authenticate/finish", webauthn_auth_finish, PUBLIC)
    r.add("POST", "/api/auth/logout", auth_logout)
    r.add("POST", "/api/auth/refresh", auth_refresh, PUBLIC)
    r.add("GET", "/api/auth/me", auth_me)
    r.add("POST", "/api/auth/mfa/totp/setup", totp_setup)
    r.add("POST", "/api/auth/mfa/totp/enable", totp_enable)
    r.add("POST", "/api/auth/mfa/webauthn/register/start", webauthn_register_start)
    r.add("POST", "/api/auth/mfa/webauthn/register/finish", webauthn_register_finish)
    r.add("GET", "/api/auth/mfa/webauthn/credentials", webauthn_list)
    r.add("DELETE", "/api/auth/mfa/webauthn/credentials/:cred", webauthn_delete)
    r.add("POST", "/api/auth/mfa/recovery/generate", recovery_generate)
    r.add("GET", "/api/auth/mfa/recovery/status", recovery_status)
    r.add("POST", "/api/auth/mfa/disable", mfa_disable)

    # ------------------------------------------------------------------ administration
    def admin_list_users(req):
        return [app.public_user(u) for u in app.users.find(limit=req.q("limit", None, int), offset=req.q("offset", 0, int),
                                                           sort="created_at")]

    def admin_create_user(req):
        email, name, password = req.need("email", "name", "password")
        return 201, app.public_user(app.create_user(email, name, password, req.json.get("role", "user")))

    def admin_get_user(req):
        return app.public_user(app.users.get(req.params["id"]))

    def admin_update_user(req):
        ch = {k: v for k, v in req.json.items() if k in ("name", "role", "approved", "email_verified")}
        if "role" in ch and ch["role"] not in A.ROLES:
            raise HttpError(400, f"role must be one of {A.ROLES}")
        if "password" in req.json:
            ch["password_hash"] = A.hash_password(req.json["password"])
        return app.public_user(app.users.update(req.params["id"], ch))

    def admin_delete_user(req):
        if req.params["id"] == req.user_id:
            raise HttpError(400, "an administrator cannot delete their own account")
        app.users.delete(req.params["id"])
        return {"deleted": True}

    def admin_stats(req):
        return {"users": app.users.count(), "runs": app.runs.runs.count(), "runs_running": app.runs.count_running(),
                "models": app.registry.models.count(), "datasets": app.datasets.col.count(),
                "endpoints": app.endpoints.col.count(), "endpoints_running": app.endpoints.count_running(),
                "notebooks": app.notebooks.col.count(), "database": app.store.health()}

    def admin_query(req):
        (collection,) = req.need("collection")
        if collection == "users":
            raise HttpError(403, "the users collection is not exposed through the query endpoint")
        if collection not in app.store.COLLECTIONS:
            raise HttpError(404, f"no collection named {collection!r} (one of {', '.join(sorted(app.store.COLLECTIONS))})")
        return app.store.query(collection, req.json.get("filter"), limit=req.json.get("limit"),
                               sort=req.json.get("sort"), descending=bool(req.json.get("descending")))

    r.add("GET", "/api/admin/users", admin_list_users, ADMIN)
    r.add("POST", "/api/admin/users", admin_create_user, ADMIN)
    r.add("GET", "/api/admin/users/:id", admin_get_user, ADMIN)
    r.add("PUT", "/api/admin/users/:id", admin_update_user, ADMIN)
    r.add("DELETE", "/api/admin/users/:id", admin_delete_user, ADMIN)
    r.add("GET", "/api/admin/stats", admin_stats, ADMIN)
    r.add("POST", "/api/admin/query", admin_query, ADMIN)
    _ = USER
