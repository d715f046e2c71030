* c1908 (c1908: 16-bit error detector / corrector): 93 gates, 1194 transistors
VDD vdd 0 DC 1.8
VIN0 nd0 0 PULSE(0 1.8 5e-10 20p 20p 1e-09 2e-09)
VIN1 nd1 0 PULSE(0 1.8 1e-09 20p 20p 2e-09 4e-09)
VIN2 nd2 0 PULSE(0 1.8 2e-09 20p 20p 4e-09 8e-09)
VIN3 nd3 0 PULSE(0 1.8 4e-09 20p 20p 8e-09 1.6e-08)
VIN4 nd4 0 PULSE(0 1.8 8e-09 20p 20p 1.6e-08 3.2e-08)
VIN5 nd5 0 PULSE(0 1.8 1.6e-08 20p 20p 3.2e-08 6.4e-08)
VIN6 nd6 0 PULSE(0 1.8 3.2e-08 20p 20p 6.4e-08 1.28e-07)
VIN7 nd7 0 PULSE(0 1.8 6.4e-08 20p 20p 1.28e-07 2.56e-07)
VIN8 nd8 0 PULSE(0 1.8 1.28e-07 20p 20p 2.56e-07 5.12e-07)
VIN9 nd9 0 PULSE(0 1.8 2.56e-07 20p 20p 5.12e-07 1.024e-06)
VIN10 nd10 0 PULSE(0 1.8 5.12e-07 20p 20p 1.024e-06 2.048e-06)
VIN11 nd11 0 PULSE(0 1.8 1.024e-06 20p 20p 2.048e-06 4.096e-06)
VIN12 nd12 0 PULSE(0 1.8 2.048e-06 20p 20p 4.096e-06 8.192e-06)
VIN13 nd13 0 PULSE(0 1.8 4.096e-06 20p 20p 8.192e-06 1.6384e-05)
VIN14 nd14 0 PULSE(0 1.8 8.192e-06 20p 20p 1.6384e-05 3.2768e-05)
VIN15 nd15 0 PULSE(0 1.8 1.6384e-05 20p 20p 3.2768e-05 6.5536e-05)
VIN16 nr0 0 PULSE(0 1.8 3.2768e-05 20p 20p 6.5536e-05 0.000131072)
VIN17 nr1 0 PULSE(0 1.8 6.5536e-05 20p 20p 0.000131072 0.000262144)
VIN18 nr2 0 PULSE(0 1.8 0.000131072 20p 20p 0.000262144 0.000524288)
VIN19 nr3 0 PULSE(0 1.8 0.000262144 20p 20p 0.000524288 0.001048576)
VIN20 nr4 0 PULSE(0 1.8 0.000524288 20p 20p 0.001048576 0.002097152)
VIN21 nen 0 PULSE(0 1.8 0.001048576 20p 20p 0.002097152 0.004194304)
CT1 t1 0 0.1f
CT2 t2 0 0.1f
CT3 t3 0 0.1f
M1 t1 nd0 vdd vdd pch w=2u l=180n
M2 t1 nd1 vdd vdd pch w=2u l=180n
CT4 t4 0 0.1f
M3 t1 nd0 t4 0 nch w=1u l=180n
M4 t4 nd1 0 0 nch w=1u l=180n
M5 t2 nd0 vdd vdd pch w=2u l=180n
M6 t2 t1 vdd vdd pch w=2u l=180n
CT5 t5 0 0.1f
M7 t2 nd0 t5 0 nch w=1u l=180n
M8 t5 t1 0 0 nch w=1u l=180n
M9 t3 nd1 vdd vdd pch w=2u l=180n
M10 t3 t1 vdd vdd pch w=2u l=180n
CT6 t6 0 0.1f
M11 t3 nd1 t6 0 nch w=1u l=180n
M12 t6 t1 0 0 nch w=1u l=180n
M13 nw1 t2 vdd vdd pch w=2u l=180n
M14 nw1 t3 vdd vdd pch w=2u l=180n
CT7 t7 0 0.1f
M15 nw1 t2 t7 0 nch w=1u l=180n
M16 t7 t3 0 0 nch w=1u l=180n
Cnw1 nw1 0 2f
CT8 t8 0 0.1f
CT9 t9 0 0.1f
CT10 t10 0 0.1f
M17 t8 nw1 vdd vdd pch w=2u l=180n
M18 t8 nd3 vdd vdd pch w=2u l=180n
CT11 t11 0 0.1f
M19 t8 nw1 t11 0 nch w=1u l=180n
M20 t11 nd3 0 0 nch w=1u l=180n
M21 t9 nw1 vdd vdd pch w=2u l=180n
M22 t9 t8 vdd vdd pch w=2u l=180n
CT12 t12 0 0.1f
M23 t9 nw1 t12 0 nch w=1u l=180n
M24 t12 t8 0 0 nch w=1u l=180n
M25 t10 nd3 vdd vdd pch w=2u l=180n
M26 t10 t8 vdd vdd pch w=2u l=180n
CT13 t13 0 0.1f
M27 t10 nd3 t13 0 nch w=1u l=180n
M28 t13 t8 0 0 nch w=1u l=180n
M29 nw2 t9 vdd vdd pch w=2u l=180n
M30 nw2 t10 vdd vdd pch w=2u l=180n
CT14 t14 0 0.1f
M31 nw2 t9 t14 0 nch w=1u l=180n
M32 t14 t10 0 0 nch w=1u l=180n
Cnw2 nw2 0 2f
CT15 t15 0 0.1f
CT16 t16 0 0.1f
CT17 t17 0 0.1f
M33 t15 nw2 vdd vdd pch w=2u l=180n
M34 t15 nd4 vdd vdd pch w=2u l=180n
CT18 t18 0 0.1f
M35 t15 nw2 t18 0 nch w=1u l=180n
M36 t18 nd4 0 0 nch w=1u l=180n
M37 t16 nw2 vdd vdd pch w=2u l=180n
M38 t16 t15 vdd vdd pch w=2u l=180n
CT19 t19 0 0.1f
M39 t16 nw2 t19 0 nch w=1u l=180n
M40 t19 t15 0 0 nch w=1u l=180n
M41 t17 nd4 vdd vdd pch w=2u l=180n
M42 t17 t15 vdd vdd pch w=2u l=180n
CT20 t20 0 0.1f
M43 t17 nd4 t20 0 nch w=1u l=180n
M44 t20 t15 0 0 nch w=1u l=180n
M45 nw3 t16 vdd vdd pch w=2u l=180n
M46 nw3 t17 vdd vdd pch w=2u l=180n
CT21 t21 0 0.1f
M47 nw3 t16 t21 0 nch w=1u l=180n
M48 t21 t17 0 0 nch w=1u l=180n
Cnw3 nw3 0 2f
CT22 t22 0 0.1f
CT23 t23 0 0.1f
CT24 t24 0 0.1f
M49 t22 nw3 vdd vdd pch w=2u l=180n
M50 t22 nd6 vdd vdd pch w=2u l=180n
CT25 t25 0 0.1f
M51 t22 nw3 t25 0 nch w=1u l=180n
M52 t25 nd6 0 0 nch w=1u l=180n
M53 t23 nw3 vdd vdd pch w=2u l=180n
M54 t23 t22 vdd vdd pch w=2u l=180n
CT26 t26 0 0.1f
M55 t23 nw3 t26 0 nch w=1u l=180n
M56 t26 t22 0 0 nch w=1u l=180n
M57 t24 nd6 vdd vdd pch w=2u l=180n
M58 t24 t22 vdd vdd pch w=2u l=180n
CT27 t27 0 0.1f
M59 t24 nd6 t27 0 nch w=1u l=180n
M60 t27 t22 0 0 nch w=1u l=180n
M61 nw4 t23 vdd vdd pch w=2u l=180n
M62 nw4 t24 vdd vdd pch w=2u l=180n
CT28 t28 0 0.1f
M63 nw4 t23 t28 0 nch w=1u l=180n
M64 t28 t24 0 0 nch w=1u l=180n
Cnw4 nw4 0 2f
CT29 t29 0 0.1f
CT30 t30 0 0.1f
CT31 t31 0 0.1f
M65 t29 nw4 vdd vdd pch w=2u l=180n
M66 t29 nd8 vdd vdd pch w=2u l=180n
CT32 t32 0 0.1f
M67 t29 nw4 t32 0 nch w=1u l=180n
M68 t32 nd8 0 0 nch w=1u l=180n
M69 t30 nw4 vdd vdd pch w=2u l=180n
M70 t30 t29 vdd vdd pch w=2u l=180n
CT33 t33 0 0.1f
M71 t30 nw4 t33 0 nch w=1u l=180n
M72 t33 t29 0 0 nch w=1u l=180n
M73 t31 nd8 vdd vdd pch w=2u l=180n
M74 t31 t29 vdd vdd pch w=2u l=180n
CT34 t34 0 0.1f
M75 t31 nd8 t34 0 nch w=1u l=180n
M76 t34 t29 0 0 nch w=1u l=180n
M77 nw5 t30 vdd vdd pch w=2u l=180n
M78 nw5 t31 vdd vdd pch w=2u l=180n
CT35 t35 0 0.1f
M79 nw5 t30 t35 0 nch w=1u l=180n
M80 t35 t31 0 0 nch w=1u l=180n
Cnw5 nw5 0 2f
CT36 t36 0 0.1f
CT37 t37 0 0.1f
CT38 t38 0 0.1f
M81 t36 nw5 vdd vdd pch w=2u l=180n
M82 t36 nd10 vdd vdd pch w=2u l=180n
CT39 t39 0 0.1f
M83 t36 nw5 t39 0 nch w=1u l=180n
M84 t39 nd10 0 0 nch w=1u l=180n
M85 t37 nw5 vdd vdd pch w=2u l=180n
M86 t37 t36 vdd vdd pch w=2u l=180n
CT40 t40 0 0.1f
M87 t37 nw5 t40 0 nch w=1u l=180n
M88 t40 t36 0 0 nch w=1u l=180n
M89 t38 nd10 vdd vdd pch w=2u l=180n
M90 t38 t36 vdd vdd pch w=2u l=180n
CT41 t41 0 0.1f
M91 t38 nd10 t41 0 nch w=1u l=180n
M92 t41 t36 0 0 nch w=1u l=180n
M93 nw6 t37 vdd vdd pch w=2u l=180n
M94 nw6 t38 vdd vdd pch w=2u l=180n
CT42 t42 0 0.1f
M95 nw6 t37 t42 0 nch w=1u l=180n
M96 t42 t38 0 0 nch w=1u l=180n
Cnw6 nw6 0 2f
CT43 t43 0 0.1f
CT44 t44 0 0.1f
CT45 t45 0 0.1f
M97 t43 nw6 vdd vdd pch w=2u l=180n
M98 t43 nd11 vdd vdd pch w=2u l=180n
CT46 t46 0 0.1f
M99 t43 nw6 t46 0 nch w=1u l=180n
M100 t46 nd11 0 0 nch w=1u l=180n
M101 t44 nw6 vdd vdd pch w=2u l=180n
M102 t44 t43 vdd vdd pch w=2u l=180n
CT47 t47 0 0.1f
M103 t44 nw6 t47 0 nch w=1u l=180n
M104 t47 t43 0 0 nch w=1u l=180n
M105 t45 nd11 vdd vdd pch w=2u l=180n
M106 t45 t43 vdd vdd pch w=2u l=180n
CT48 t48 0 0.1f
M107 t45 nd11 t48 0 nch w=1u l=180n
M108 t48 t43 0 0 nch w=1u l=180n
M109 nw7 t44 vdd vdd pch w=2u l=180n
M110 nw7 t45 vdd vdd pch w=2u l=180n
CT49 t49 0 0.1f
M111 nw7 t44 t49 0 nch w=1u l=180n
M112 t49 t45 0 0 nch w=1u l=180n
Cnw7 nw7 0 2f
CT50 t50 0 0.1f
CT51 t51 0 0.1f
CT52 t52 0 0.1f
M113 t50 nw7 vdd vdd pch w=2u l=180n
M114 t50 nd13 vdd vdd pch w=2u l=180n
CT53 t53 0 0.1f
M115 t50 nw7 t53 0 nch w=1u l=180n
M116 t53 nd13 0 0 nch w=1u l=180n
M117 t51 nw7 vdd vdd pch w=2u l=180n
M118 t51 t50 vdd vdd pch w=2u l=180n
CT54 t54 0 0.1f
M119 t51 nw7 t54 0 nch w=1u l=180n
M120 t54 t50 0 0 nch w=1u l=180n
M121 t52 nd13 vdd vdd pch w=2u l=180n
M122 t52 t50 vdd vdd pch w=2u l=180n
CT55 t55 0 0.1f
M123 t52 nd13 t55 0 nch w=1u l=180n
M124 t55 t50 0 0 nch w=1u l=180n
M125 nw8 t51 vdd vdd pch w=2u l=180n
M126 nw8 t52 vdd vdd pch w=2u l=180n
CT56 t56 0 0.1f
M127 nw8 t51 t56 0 nch w=1u l=180n
M128 t56 t52 0 0 nch w=1u l=180n
Cnw8 nw8 0 2f
CT57 t57 0 0.1f
CT58 t58 0 0.1f
CT59 t59 0 0.1f
M129 t57 nw8 vdd vdd pch w=2u l=180n
M130 t57 nd15 vdd vdd pch w=2u l=180n
CT60 t60 0 0.1f
M131 t57 nw8 t60 0 nch w=1u l=180n
M132 t60 nd15 0 0 nch w=1u l=180n
M133 t58 nw8 vdd vdd pch w=2u l=180n
M134 t58 t57 vdd vdd pch w=2u l=180n
CT61 t61 0 0.1f
M135 t58 nw8 t61 0 nch w=1u l=180n
M136 t61 t57 0 0 nch w=1u l=180n
M137 t59 nd15 vdd vdd pch w=2u l=180n
M138 t59 t57 vdd vdd pch w=2u l=180n
CT62 t62 0 0.1f
M139 t59 nd15 t62 0 nch w=1u l=180n
M140 t62 t57 0 0 nch w=1u l=180n
M141 nw9 t58 vdd vdd pch w=2u l=180n
M142 nw9 t59 vdd vdd pch w=2u l=180n
CT63 t63 0 0.1f
M143 nw9 t58 t63 0 nch w=1u l=180n
M144 t63 t59 0 0 nch w=1u l=180n
Cnw9 nw9 0 2f
CT64 t64 0 0.1f
CT65 t65 0 0.1f
CT66 t66 0 0.1f
M145 t64 nw9 vdd vdd pch w=2u l=180n
M146 t64 nr0 vdd vdd pch w=2u l=180n
CT67 t67 0 0.1f
M147 t64 nw9 t67 0 nch w=1u l=180n
M148 t67 nr0 0 0 nch w=1u l=180n
M149 t65 nw9 vdd vdd pch w=2u l=180n
M150 t65 t64 vdd vdd pch w=2u l=180n
CT68 t68 0 0.1f
M151 t65 nw9 t68 0 nch w=1u l=180n
M152 t68 t64 0 0 nch w=1u l=180n
M153 t66 nr0 vdd vdd pch w=2u l=180n
M154 t66 t64 vdd vdd pch w=2u l=180n
CT69 t69 0 0.1f
M155 t66 nr0 t69 0 nch w=1u l=180n
M156 t69 t64 0 0 nch w=1u l=180n
M157 nw10 t65 vdd vdd pch w=2u l=180n
M158 nw10 t66 vdd vdd pch w=2u l=180n
CT70 t70 0 0.1f
M159 nw10 t65 t70 0 nch w=1u l=180n
M160 t70 t66 0 0 nch w=1u l=180n
Cnw10 nw10 0 2f
CT71 t71 0 0.1f
CT72 t72 0 0.1f
CT73 t73 0 0.1f
M161 t71 nd0 vdd vdd pch w=2u l=180n
M162 t71 nd2 vdd vdd pch w=2u l=180n
CT74 t74 0 0.1f
M163 t71 nd0 t74 0 nch w=1u l=180n
M164 t74 nd2 0 0 nch w=1u l=180n
M165 t72 nd0 vdd vdd pch w=2u l=180n
M166 t72 t71 vdd vdd pch w=2u l=180n
CT75 t75 0 0.1f
M167 t72 nd0 t75 0 nch w=1u l=180n
M168 t75 t71 0 0 nch w=1u l=180n
M169 t73 nd2 vdd vdd pch w=2u l=180n
M170 t73 t71 vdd vdd pch w=2u l=180n
CT76 t76 0 0.1f
M171 t73 nd2 t76 0 nch w=1u l=180n
M172 t76 t71 0 0 nch w=1u l=180n
M173 nw11 t72 vdd vdd pch w=2u l=180n
M174 nw11 t73 vdd vdd pch w=2u l=180n
CT77 t77 0 0.1f
M175 nw11 t72 t77 0 nch w=1u l=180n
M176 t77 t73 0 0 nch w=1u l=180n
Cnw11 nw11 0 2f
CT78 t78 0 0.1f
CT79 t79 0 0.1f
CT80 t80 0 0.1f
M177 t78 nw11 vdd vdd pch w=2u l=180n
M178 t78 nd3 vdd vdd pch w=2u l=180n
CT81 t81 0 0.1f
M179 t78 nw11 t81 0 nch w=1u l=180n
M180 t81 nd3 0 0 nch w=1u l=180n
M181 t79 nw11 vdd vdd pch w=2u l=180n
M182 t79 t78 vdd vdd pch w=2u l=180n
CT82 t82 0 0.1f
M183 t79 nw11 t82 0 nch w=1u l=180n
M184 t82 t78 0 0 nch w=1u l=180n
M185 t80 nd3 vdd vdd pch w=2u l=180n
M186 t80 t78 vdd vdd pch w=2u l=180n
CT83 t83 0 0.1f
M187 t80 nd3 t83 0 nch w=1u l=180n
M188 t83 t78 0 0 nch w=1u l=180n
M189 nw12 t79 vdd vdd pch w=2u l=180n
M190 nw12 t80 vdd vdd pch w=2u l=180n
CT84 t84 0 0.1f
M191 nw12 t79 t84 0 nch w=1u l=180n
M192 t84 t80 0 0 nch w=1u l=180n
Cnw12 nw12 0 2f
CT85 t85 0 0.1f
CT86 t86 0 0.1f
CT87 t87 0 0.1f
M193 t85 nw12 vdd vdd pch w=2u l=180n
M194 t85 nd5 vdd vdd pch w=2u l=180n
CT88 t88 0 0.1f
M195 t85 nw12 t88 0 nch w=1u l=180n
M196 t88 nd5 0 0 nch w=1u l=180n
M197 t86 nw12 vdd vdd pch w=2u l=180n
M198 t86 t85 vdd vdd pch w=2u l=180n
CT89 t89 0 0.1f
M199 t86 nw12 t89 0 nch w=1u l=180n
M200 t89 t85 0 0 nch w=1u l=180n
M201 t87 nd5 vdd vdd pch w=2u l=180n
M202 t87 t85 vdd vdd pch w=2u l=180n
CT90 t90 0 0.1f
M203 t87 nd5 t90 0 nch w=1u l=180n
M204 t90 t85 0 0 nch w=1u l=180n
M205 nw13 t86 vdd vdd pch w=2u l=180n
M206 nw13 t87 vdd vdd pch w=2u l=180n
CT91 t91 0 0.1f
M207 nw13 t86 t91 0 nch w=1u l=180n
M208 t91 t87 0 0 nch w=1u l=180n
Cnw13 nw13 0 2f
CT92 t92 0 0.1f
CT93 t93 0 0.1f
CT94 t94 0 0.1f
M209 t92 nw13 vdd vdd pch w=2u l=180n
M210 t92 nd6 vdd vdd pch w=2u l=180n
CT95 t95 0 0.1f
M211 t92 nw13 t95 0 nch w=1u l=180n
M212 t95 nd6 0 0 nch w=1u l=180n
M213 t93 nw13 vdd vdd pch w=2u l=180n
M214 t93 t92 vdd vdd pch w=2u l=180n
CT96 t96 0 0.1f
M215 t93 nw13 t96 0 nch w=1u l=180n
M216 t96 t92 0 0 nch w=1u l=180n
M217 t94 nd6 vdd vdd pch w=2u l=180n
M218 t94 t92 vdd vdd pch w=2u l=180n
CT97 t97 0 0.1f
M219 t94 nd6 t97 0 nch w=1u l=180n
M220 t97 t92 0 0 nch w=1u l=180n
M221 nw14 t93 vdd vdd pch w=2u l=180n
M222 nw14 t94 vdd vdd pch w=2u l=180n
CT98 t98 0 0.1f
M223 nw14 t93 t98 0 nch w=1u l=180n
M224 t98 t94 0 0 nch w=1u l=180n
Cnw14 nw14 0 2f
CT99 t99 0 0.1f
CT100 t100 0 0.1f
CT101 t101 0 0.1f
M225 t99 nw14 vdd vdd pch w=2u l=180n
M226 t99 nd9 vdd vdd pch w=2u l=180n
CT102 t102 0 0.1f
M227 t99 nw14 t102 0 nch w=1u l=180n
M228 t102 nd9 0 0 nch w=1u l=180n
M229 t100 nw14 vdd vdd pch w=2u l=180n
M230 t100 t99 vdd vdd pch w=2u l=180n
CT103 t103 0 0.1f
M231 t100 nw14 t103 0 nch w=1u l=180n
M232 t103 t99 0 0 nch w=1u l=180n
M233 t101 nd9 vdd vdd pch w=2u l=180n
M234 t101 t99 vdd vdd pch w=2u l=180n
CT104 t104 0 0.1f
M235 t101 nd9 t104 0 nch w=1u l=180n
M236 t104 t99 0 0 nch w=1u l=180n
M237 nw15 t100 vdd vdd pch w=2u l=180n
M238 nw15 t101 vdd vdd pch w=2u l=180n
CT105 t105 0 0.1f
M239 nw15 t100 t105 0 nch w=1u l=180n
M240 t105 t101 0 0 nch w=1u l=180n
Cnw15 nw15 0 2f
CT106 t106 0 0.1f
CT107 t107 0 0.1f
CT108 t108 0 0.1f
M241 t106 nw15 vdd vdd pch w=2u l=180n
M242 t106 nd10 vdd vdd pch w=2u l=180n
CT109 t109 0 0.1f
M243 t106 nw15 t109 0 nch w=1u l=180n
M244 t109 nd10 0 0 nch w=1u l=180n
M245 t107 nw15 vdd vdd pch w=2u l=180n
M246 t107 t106 vdd vdd pch w=2u l=180n
CT110 t110 0 0.1f
M247 t107 nw15 t110 0 nch w=1u l=180n
M248 t110 t106 0 0 nch w=1u l=180n
M249 t108 nd10 vdd vdd pch w=2u l=180n
M250 t108 t106 vdd vdd pch w=2u l=180n
CT111 t111 0 0.1f
M251 t108 nd10 t111 0 nch w=1u l=180n
M252 t111 t106 0 0 nch w=1u l=180n
M253 nw16 t107 vdd vdd pch w=2u l=180n
M254 nw16 t108 vdd vdd pch w=2u l=180n
CT112 t112 0 0.1f
M255 nw16 t107 t112 0 nch w=1u l=180n
M256 t112 t108 0 0 nch w=1u l=180n
Cnw16 nw16 0 2f
CT113 t113 0 0.1f
CT114 t114 0 0.1f
CT115 t115 0 0.1f
M257 t113 nw16 vdd vdd pch w=2u l=180n
M258 t113 nd12 vdd vdd pch w=2u l=180n
CT116 t116 0 0.1f
M259 t113 nw16 t116 0 nch w=1u l=180n
M260 t116 nd12 0 0 nch w=1u l=180n
M261 t114 nw16 vdd vdd pch w=2u l=180n
M262 t114 t113 vdd vdd pch w=2u l=180n
CT117 t117 0 0.1f
M263 t114 nw16 t117 0 nch w=1u l=180n
M264 t117 t113 0 0 nch w=1u l=180n
M265 t115 nd12 vdd vdd pch w=2u l=180n
M266 t115 t113 vdd vdd pch w=2u l=180n
CT118 t118 0 0.1f
M267 t115 nd12 t118 0 nch w=1u l=180n
M268 t118 t113 0 0 nch w=1u l=180n
M269 nw17 t114 vdd vdd pch w=2u l=180n
M270 nw17 t115 vdd vdd pch w=2u l=180n
CT119 t119 0 0.1f
M271 nw17 t114 t119 0 nch w=1u l=180n
M272 t119 t115 0 0 nch w=1u l=180n
Cnw17 nw17 0 2f
CT120 t120 0 0.1f
CT121 t121 0 0.1f
CT122 t122 0 0.1f
M273 t120 nw17 vdd vdd pch w=2u l=180n
M274 t120 nd13 vdd vdd pch w=2u l=180n
CT123 t123 0 0.1f
M275 t120 nw17 t123 0 nch w=1u l=180n
M276 t123 nd13 0 0 nch w=1u l=180n
M277 t121 nw17 vdd vdd pch w=2u l=180n
M278 t121 t120 vdd vdd pch w=2u l=180n
CT124 t124 0 0.1f
M279 t121 nw17 t124 0 nch w=1u l=180n
M280 t124 t120 0 0 nch w=1u l=180n
M281 t122 nd13 vdd vdd pch w=2u l=180n
M282 t122 t120 vdd vdd pch w=2u l=180n
CT125 t125 0 0.1f
M283 t122 nd13 t125 0 nch w=1u l=180n
M284 t125 t120 0 0 nch w=1u l=180n
M285 nw18 t121 vdd vdd pch w=2u l=180n
M286 nw18 t122 vdd vdd pch w=2u l=180n
CT126 t126 0 0.1f
M287 nw18 t121 t126 0 nch w=1u l=180n
M288 t126 t122 0 0 nch w=1u l=180n
Cnw18 nw18 0 2f
CT127 t127 0 0.1f
CT128 t128 0 0.1f
CT129 t129 0 0.1f
M289 t127 nw18 vdd vdd pch w=2u l=180n
M290 t127 nr1 vdd vdd pch w=2u l=180n
CT130 t130 0 0.1f
M291 t127 nw18 t130 0 nch w=1u l=180n
M292 t130 nr1 0 0 nch w=1u l=180n
M293 t128 nw18 vdd vdd pch w=2u l=180n
M294 t128 t127 vdd vdd pch w=2u l=180n
CT131 t131 0 0.1f
M295 t128 nw18 t131 0 nch w=1u l=180n
M296 t131 t127 0 0 nch w=1u l=180n
M297 t129 nr1 vdd vdd pch w=2u l=180n
M298 t129 t127 vdd vdd pch w=2u l=180n
CT132 t132 0 0.1f
M299 t129 nr1 t132 0 nch w=1u l=180n
M300 t132 t127 0 0 nch w=1u l=180n
M301 nw19 t128 vdd vdd pch w=2u l=180n
M302 nw19 t129 vdd vdd pch w=2u l=180n
CT133 t133 0 0.1f
M303 nw19 t128 t133 0 nch w=1u l=180n
M304 t133 t129 0 0 nch w=1u l=180n
Cnw19 nw19 0 2f
CT134 t134 0 0.1f
CT135 t135 0 0.1f
CT136 t136 0 0.1f
M305 t134 nd1 vdd vdd pch w=2u l=180n
M306 t134 nd2 vdd vdd pch w=2u l=180n
CT137 t137 0 0.1f
M307 t134 nd1 t137 0 nch w=1u l=180n
M308 t137 nd2 0 0 nch w=1u l=180n
M309 t135 nd1 vdd vdd pch w=2u l=180n
M310 t135 t134 vdd vdd pch w=2u l=180n
CT138 t138 0 0.1f
M311 t135 nd1 t138 0 nch w=1u l=180n
M312 t138 t134 0 0 nch w=1u l=180n
M313 t136 nd2 vdd vdd pch w=2u l=180n
M314 t136 t134 vdd vdd pch w=2u l=180n
CT139 t139 0 0.1f
M315 t136 nd2 t139 0 nch w=1u l=180n
M316 t139 t134 0 0 nch w=1u l=180n
M317 nw20 t135 vdd vdd pch w=2u l=180n
M318 nw20 t136 vdd vdd pch w=2u l=180n
CT140 t140 0 0.1f
M319 nw20 t135 t140 0 nch w=1u l=180n
M320 t140 t136 0 0 nch w=1u l=180n
Cnw20 nw20 0 2f
CT141 t141 0 0.1f
CT142 t142 0 0.1f
CT143 t143 0 0.1f
M321 t141 nw20 vdd vdd pch w=2u l=180n
M322 t141 nd3 vdd vdd pch w=2u l=180n
CT144 t144 0 0.1f
M323 t141 nw20 t144 0 nch w=1u l=180n
M324 t144 nd3 0 0 nch w=1u l=180n
M325 t142 nw20 vdd vdd pch w=2u l=180n
M326 t142 t141 vdd vdd pch w=2u l=180n
CT145 t145 0 0.1f
M327 t142 nw20 t145 0 nch w=1u l=180n
M328 t145 t141 0 0 nch w=1u l=180n
M329 t143 nd3 vdd vdd pch w=2u l=180n
M330 t143 t141 vdd vdd pch w=2u l=180n
CT146 t146 0 0.1f
M331 t143 nd3 t146 0 nch w=1u l=180n
M332 t146 t141 0 0 nch w=1u l=180n
M333 nw21 t142 vdd vdd pch w=2u l=180n
M334 nw21 t143 vdd vdd pch w=2u l=180n
CT147 t147 0 0.1f
M335 nw21 t142 t147 0 nch w=1u l=180n
M336 t147 t143 0 0 nch w=1u l=180n
Cnw21 nw21 0 2f
CT148 t148 0 0.1f
CT149 t149 0 0.1f
CT150 t150 0 0.1f
M337 t148 nw21 vdd vdd pch w=2u l=180n
M338 t148 nd7 vdd vdd pch w=2u l=180n
CT151 t151 0 0.1f
M339 t148 nw21 t151 0 nch w=1u l=180n
M340 t151 nd7 0 0 nch w=1u l=180n
M341 t149 nw21 vdd vdd pch w=2u l=180n
M342 t149 t148 vdd vdd pch w=2u l=180n
CT152 t152 0 0.1f
M343 t149 nw21 t152 0 nch w=1u l=180n
M344 t152 t148 0 0 nch w=1u l=180n
M345 t150 nd7 vdd vdd pch w=2u l=180n
M346 t150 t148 vdd vdd pch w=2u l=180n
CT153 t153 0 0.1f
M347 t150 nd7 t153 0 nch w=1u l=180n
M348 t153 t148 0 0 nch w=1u l=180n
M349 nw22 t149 vdd vdd pch w=2u l=180n
M350 nw22 t150 vdd vdd pch w=2u l=180n
CT154 t154 0 0.1f
M351 nw22 t149 t154 0 nch w=1u l=180n
M352 t154 t150 0 0 nch w=1u l=180n
Cnw22 nw22 0 2f
CT155 t155 0 0.1f
CT156 t156 0 0.1f
CT157 t157 0 0.1f
M353 t155 nw22 vdd vdd pch w=2u l=180n
M354 t155 nd8 vdd vdd pch w=2u l=180n
CT158 t158 0 0.1f
M355 t155 nw22 t158 0 nch w=1u l=180n
M356 t158 nd8 0 0 nch w=1u l=180n
M357 t156 nw22 vdd vdd pch w=2u l=180n
M358 t156 t155 vdd vdd pch w=2u l=180n
CT159 t159 0 0.1f
M359 t156 nw22 t159 0 nch w=1u l=180n
M360 t159 t155 0 0 nch w=1u l=180n
M361 t157 nd8 vdd vdd pch w=2u l=180n
M362 t157 t155 vdd vdd pch w=2u l=180n
CT160 t160 0 0.1f
M363 t157 nd8 t160 0 nch w=1u l=180n
M364 t160 t155 0 0 nch w=1u l=180n
M365 nw23 t156 vdd vdd pch w=2u l=180n
M366 nw23 t157 vdd vdd pch w=2u l=180n
CT161 t161 0 0.1f
M367 nw23 t156 t161 0 nch w=1u l=180n
M368 t161 t157 0 0 nch w=1u l=180n
Cnw23 nw23 0 2f
CT162 t162 0 0.1f
CT163 t163 0 0.1f
CT164 t164 0 0.1f
M369 t162 nw23 vdd vdd pch w=2u l=180n
M370 t162 nd9 vdd vdd pch w=2u l=180n
CT165 t165 0 0.1f
M371 t162 nw23 t165 0 nch w=1u l=180n
M372 t165 nd9 0 0 nch w=1u l=180n
M373 t163 nw23 vdd vdd pch w=2u l=180n
M374 t163 t162 vdd vdd pch w=2u l=180n
CT166 t166 0 0.1f
M375 t163 nw23 t166 0 nch w=1u l=180n
M376 t166 t162 0 0 nch w=1u l=180n
M377 t164 nd9 vdd vdd pch w=2u l=180n
M378 t164 t162 vdd vdd pch w=2u l=180n
CT167 t167 0 0.1f
M379 t164 nd9 t167 0 nch w=1u l=180n
M380 t167 t162 0 0 nch w=1u l=180n
M381 nw24 t163 vdd vdd pch w=2u l=180n
M382 nw24 t164 vdd vdd pch w=2u l=180n
CT168 t168 0 0.1f
M383 nw24 t163 t168 0 nch w=1u l=180n
M384 t168 t164 0 0 nch w=1u l=180n
Cnw24 nw24 0 2f
CT169 t169 0 0.1f
CT170 t170 0 0.1f
CT171 t171 0 0.1f
M385 t169 nw24 vdd vdd pch w=2u l=180n
M386 t169 nd10 vdd vdd pch w=2u l=180n
CT172 t172 0 0.1f
M387 t169 nw24 t172 0 nch w=1u l=180n
M388 t172 nd10 0 0 nch w=1u l=180n
M389 t170 nw24 vdd vdd pch w=2u l=180n
M390 t170 t169 vdd vdd pch w=2u l=180n
CT173 t173 0 0.1f
M391 t170 nw24 t173 0 nch w=1u l=180n
M392 t173 t169 0 0 nch w=1u l=180n
M393 t171 nd10 vdd vdd pch w=2u l=180n
M394 t171 t169 vdd vdd pch w=2u l=180n
CT174 t174 0 0.1f
M395 t171 nd10 t174 0 nch w=1u l=180n
M396 t174 t169 0 0 nch w=1u l=180n
M397 nw25 t170 vdd vdd pch w=2u l=180n
M398 nw25 t171 vdd vdd pch w=2u l=180n
CT175 t175 0 0.1f
M399 nw25 t170 t175 0 nch w=1u l=180n
M400 t175 t171 0 0 nch w=1u l=180n
Cnw25 nw25 0 2f
CT176 t176 0 0.1f
CT177 t177 0 0.1f
CT178 t178 0 0.1f
M401 t176 nw25 vdd vdd pch w=2u l=180n
M402 t176 nd14 vdd vdd pch w=2u l=180n
CT179 t179 0 0.1f
M403 t176 nw25 t179 0 nch w=1u l=180n
M404 t179 nd14 0 0 nch w=1u l=180n
M405 t177 nw25 vdd vdd pch w=2u l=180n
M406 t177 t176 vdd vdd pch w=2u l=180n
CT180 t180 0 0.1f
M407 t177 nw25 t180 0 nch w=1u l=180n
M408 t180 t176 0 0 nch w=1u l=180n
M409 t178 nd14 vdd vdd pch w=2u l=180n
M410 t178 t176 vdd vdd pch w=2u l=180n
CT181 t181 0 0.1f
M411 t178 nd14 t181 0 nch w=1u l=180n
M412 t181 t176 0 0 nch w=1u l=180n
M413 nw26 t177 vdd vdd pch w=2u l=180n
M414 nw26 t178 vdd vdd pch w=2u l=180n
CT182 t182 0 0.1f
M415 nw26 t177 t182 0 nch w=1u l=180n
M416 t182 t178 0 0 nch w=1u l=180n
Cnw26 nw26 0 2f
CT183 t183 0 0.1f
CT184 t184 0 0.1f
CT185 t185 0 0.1f
M417 t183 nw26 vdd vdd pch w=2u l=180n
M418 t183 nd15 vdd vdd pch w=2u l=180n
CT186 t186 0 0.1f
M419 t183 nw26 t186 0 nch w=1u l=180n
M420 t186 nd15 0 0 nch w=1u l=180n
M421 t184 nw26 vdd vdd pch w=2u l=180n
M422 t184 t183 vdd vdd pch w=2u l=180n
CT187 t187 0 0.1f
M423 t184 nw26 t187 0 nch w=1u l=180n
M424 t187 t183 0 0 nch w=1u l=180n
M425 t185 nd15 vdd vdd pch w=2u l=180n
M426 t185 t183 vdd vdd pch w=2u l=180n
CT188 t188 0 0.1f
M427 t185 nd15 t188 0 nch w=1u l=180n
M428 t188 t183 0 0 nch w=1u l=180n
M429 nw27 t184 vdd vdd pch w=2u l=180n
M430 nw27 t185 vdd vdd pch w=2u l=180n
CT189 t189 0 0.1f
M431 nw27 t184 t189 0 nch w=1u l=180n
M432 t189 t185 0 0 nch w=1u l=180n
Cnw27 nw27 0 2f
CT190 t190 0 0.1f
CT191 t191 0 0.1f
CT192 t192 0 0.1f
M433 t190 nw27 vdd vdd pch w=2u l=180n
M434 t190 nr2 vdd vdd pch w=2u l=180n
CT193 t193 0 0.1f
M435 t190 nw27 t193 0 nch w=1u l=180n
M436 t193 nr2 0 0 nch w=1u l=180n
M437 t191 nw27 vdd vdd pch w=2u l=180n
M438 t191 t190 vdd vdd pch w=2u l=180n
CT194 t194 0 0.1f
M439 t191 nw27 t194 0 nch w=1u l=180n
M440 t194 t190 0 0 nch w=1u l=180n
M441 t192 nr2 vdd vdd pch w=2u l=180n
M442 t192 t190 vdd vdd pch w=2u l=180n
CT195 t195 0 0.1f
M443 t192 nr2 t195 0 nch w=1u l=180n
M444 t195 t190 0 0 nch w=1u l=180n
M445 nw28 t191 vdd vdd pch w=2u l=180n
M446 nw28 t192 vdd vdd pch w=2u l=180n
CT196 t196 0 0.1f
M447 nw28 t191 t196 0 nch w=1u l=180n
M448 t196 t192 0 0 nch w=1u l=180n
Cnw28 nw28 0 2f
CT197 t197 0 0.1f
CT198 t198 0 0.1f
CT199 t199 0 0.1f
M449 t197 nd4 vdd vdd pch w=2u l=180n
M450 t197 nd5 vdd vdd pch w=2u l=180n
CT200 t200 0 0.1f
M451 t197 nd4 t200 0 nch w=1u l=180n
M452 t200 nd5 0 0 nch w=1u l=180n
M453 t198 nd4 vdd vdd pch w=2u l=180n
M454 t198 t197 vdd vdd pch w=2u l=180n
CT201 t201 0 0.1f
M455 t198 nd4 t201 0 nch w=1u l=180n
M456 t201 t197 0 0 nch w=1u l=180n
M457 t199 nd5 vdd vdd pch w=2u l=180n
M458 t199 t197 vdd vdd pch w=2u l=180n
CT202 t202 0 0.1f
M459 t199 nd5 t202 0 nch w=1u l=180n
M460 t202 t197 0 0 nch w=1u l=180n
M461 nw29 t198 vdd vdd pch w=2u l=180n
M462 nw29 t199 vdd vdd pch w=2u l=180n
CT203 t203 0 0.1f
M463 nw29 t198 t203 0 nch w=1u l=180n
M464 t203 t199 0 0 nch w=1u l=180n
Cnw29 nw29 0 2f
CT204 t204 0 0.1f
CT205 t205 0 0.1f
CT206 t206 0 0.1f
M465 t204 nw29 vdd vdd pch w=2u l=180n
M466 t204 nd6 vdd vdd pch w=2u l=180n
CT207 t207 0 0.1f
M467 t204 nw29 t207 0 nch w=1u l=180n
M468 t207 nd6 0 0 nch w=1u l=180n
M469 t205 nw29 vdd vdd pch w=2u l=180n
M470 t205 t204 vdd vdd pch w=2u l=180n
CT208 t208 0 0.1f
M471 t205 nw29 t208 0 nch w=1u l=180n
M472 t208 t204 0 0 nch w=1u l=180n
M473 t206 nd6 vdd vdd pch w=2u l=180n
M474 t206 t204 vdd vdd pch w=2u l=180n
CT209 t209 0 0.1f
M475 t206 nd6 t209 0 nch w=1u l=180n
M476 t209 t204 0 0 nch w=1u l=180n
M477 nw30 t205 vdd vdd pch w=2u l=180n
M478 nw30 t206 vdd vdd pch w=2u l=180n
CT210 t210 0 0.1f
M479 nw30 t205 t210 0 nch w=1u l=180n
M480 t210 t206 0 0 nch w=1u l=180n
Cnw30 nw30 0 2f
CT211 t211 0 0.1f
CT212 t212 0 0.1f
CT213 t213 0 0.1f
M481 t211 nw30 vdd vdd pch w=2u l=180n
M482 t211 nd7 vdd vdd pch w=2u l=180n
CT214 t214 0 0.1f
M483 t211 nw30 t214 0 nch w=1u l=180n
M484 t214 nd7 0 0 nch w=1u l=180n
M485 t212 nw30 vdd vdd pch w=2u l=180n
M486 t212 t211 vdd vdd pch w=2u l=180n
CT215 t215 0 0.1f
M487 t212 nw30 t215 0 nch w=1u l=180n
M488 t215 t211 0 0 nch w=1u l=180n
M489 t213 nd7 vdd vdd pch w=2u l=180n
M490 t213 t211 vdd vdd pch w=2u l=180n
CT216 t216 0 0.1f
M491 t213 nd7 t216 0 nch w=1u l=180n
M492 t216 t211 0 0 nch w=1u l=180n
M493 nw31 t212 vdd vdd pch w=2u l=180n
M494 nw31 t213 vdd vdd pch w=2u l=180n
CT217 t217 0 0.1f
M495 nw31 t212 t217 0 nch w=1u l=180n
M496 t217 t213 0 0 nch w=1u l=180n
Cnw31 nw31 0 2f
CT218 t218 0 0.1f
CT219 t219 0 0.1f
CT220 t220 0 0.1f
M497 t218 nw31 vdd vdd pch w=2u l=180n
M498 t218 nd8 vdd vdd pch w=2u l=180n
CT221 t221 0 0.1f
M499 t218 nw31 t221 0 nch w=1u l=180n
M500 t221 nd8 0 0 nch w=1u l=180n
M501 t219 nw31 vdd vdd pch w=2u l=180n
M502 t219 t218 vdd vdd pch w=2u l=180n
CT222 t222 0 0.1f
M503 t219 nw31 t222 0 nch w=1u l=180n
M504 t222 t218 0 0 nch w=1u l=180n
M505 t220 nd8 vdd vdd pch w=2u l=180n
M506 t220 t218 vdd vdd pch w=2u l=180n
CT223 t223 0 0.1f
M507 t220 nd8 t223 0 nch w=1u l=180n
M508 t223 t218 0 0 nch w=1u l=180n
M509 nw32 t219 vdd vdd pch w=2u l=180n
M510 nw32 t220 vdd vdd pch w=2u l=180n
CT224 t224 0 0.1f
M511 nw32 t219 t224 0 nch w=1u l=180n
M512 t224 t220 0 0 nch w=1u l=180n
Cnw32 nw32 0 2f
CT225 t225 0 0.1f
CT226 t226 0 0.1f
CT227 t227 0 0.1f
M513 t225 nw32 vdd vdd pch w=2u l=180n
M514 t225 nd9 vdd vdd pch w=2u l=180n
CT228 t228 0 0.1f
M515 t225 nw32 t228 0 nch w=1u l=180n
M516 t228 nd9 0 0 nch w=1u l=180n
M517 t226 nw32 vdd vdd pch w=2u l=180n
M518 t226 t225 vdd vdd pch w=2u l=180n
CT229 t229 0 0.1f
M519 t226 nw32 t229 0 nch w=1u l=180n
M520 t229 t225 0 0 nch w=1u l=180n
M521 t227 nd9 vdd vdd pch w=2u l=180n
M522 t227 t225 vdd vdd pch w=2u l=180n
CT230 t230 0 0.1f
M523 t227 nd9 t230 0 nch w=1u l=180n
M524 t230 t225 0 0 nch w=1u l=180n
M525 nw33 t226 vdd vdd pch w=2u l=180n
M526 nw33 t227 vdd vdd pch w=2u l=180n
CT231 t231 0 0.1f
M527 nw33 t226 t231 0 nch w=1u l=180n
M528 t231 t227 0 0 nch w=1u l=180n
Cnw33 nw33 0 2f
CT232 t232 0 0.1f
CT233 t233 0 0.1f
CT234 t234 0 0.1f
M529 t232 nw33 vdd vdd pch w=2u l=180n
M530 t232 nd10 vdd vdd pch w=2u l=180n
CT235 t235 0 0.1f
M531 t232 nw33 t235 0 nch w=1u l=180n
M532 t235 nd10 0 0 nch w=1u l=180n
M533 t233 nw33 vdd vdd pch w=2u l=180n
M534 t233 t232 vdd vdd pch w=2u l=180n
CT236 t236 0 0.1f
M535 t233 nw33 t236 0 nch w=1u l=180n
M536 t236 t232 0 0 nch w=1u l=180n
M537 t234 nd10 vdd vdd pch w=2u l=180n
M538 t234 t232 vdd vdd pch w=2u l=180n
CT237 t237 0 0.1f
M539 t234 nd10 t237 0 nch w=1u l=180n
M540 t237 t232 0 0 nch w=1u l=180n
M541 nw34 t233 vdd vdd pch w=2u l=180n
M542 nw34 t234 vdd vdd pch w=2u l=180n
CT238 t238 0 0.1f
M543 nw34 t233 t238 0 nch w=1u l=180n
M544 t238 t234 0 0 nch w=1u l=180n
Cnw34 nw34 0 2f
CT239 t239 0 0.1f
CT240 t240 0 0.1f
CT241 t241 0 0.1f
M545 t239 nw34 vdd vdd pch w=2u l=180n
M546 t239 nr3 vdd vdd pch w=2u l=180n
CT242 t242 0 0.1f
M547 t239 nw34 t242 0 nch w=1u l=180n
M548 t242 nr3 0 0 nch w=1u l=180n
M549 t240 nw34 vdd vdd pch w=2u l=180n
M550 t240 t239 vdd vdd pch w=2u l=180n
CT243 t243 0 0.1f
M551 t240 nw34 t243 0 nch w=1u l=180n
M552 t243 t239 0 0 nch w=1u l=180n
M553 t241 nr3 vdd vdd pch w=2u l=180n
M554 t241 t239 vdd vdd pch w=2u l=180n
CT244 t244 0 0.1f
M555 t241 nr3 t244 0 nch w=1u l=180n
M556 t244 t239 0 0 nch w=1u l=180n
M557 nw35 t240 vdd vdd pch w=2u l=180n
M558 nw35 t241 vdd vdd pch w=2u l=180n
CT245 t245 0 0.1f
M559 nw35 t240 t245 0 nch w=1u l=180n
M560 t245 t241 0 0 nch w=1u l=180n
Cnw35 nw35 0 2f
CT246 t246 0 0.1f
CT247 t247 0 0.1f
CT248 t248 0 0.1f
M561 t246 nd11 vdd vdd pch w=2u l=180n
M562 t246 nd12 vdd vdd pch w=2u l=180n
CT249 t249 0 0.1f
M563 t246 nd11 t249 0 nch w=1u l=180n
M564 t249 nd12 0 0 nch w=1u l=180n
M565 t247 nd11 vdd vdd pch w=2u l=180n
M566 t247 t246 vdd vdd pch w=2u l=180n
CT250 t250 0 0.1f
M567 t247 nd11 t250 0 nch w=1u l=180n
M568 t250 t246 0 0 nch w=1u l=180n
M569 t248 nd12 vdd vdd pch w=2u l=180n
M570 t248 t246 vdd vdd pch w=2u l=180n
CT251 t251 0 0.1f
M571 t248 nd12 t251 0 nch w=1u l=180n
M572 t251 t246 0 0 nch w=1u l=180n
M573 nw36 t247 vdd vdd pch w=2u l=180n
M574 nw36 t248 vdd vdd pch w=2u l=180n
CT252 t252 0 0.1f
M575 nw36 t247 t252 0 nch w=1u l=180n
M576 t252 t248 0 0 nch w=1u l=180n
Cnw36 nw36 0 2f
CT253 t253 0 0.1f
CT254 t254 0 0.1f
CT255 t255 0 0.1f
M577 t253 nw36 vdd vdd pch w=2u l=180n
M578 t253 nd13 vdd vdd pch w=2u l=180n
CT256 t256 0 0.1f
M579 t253 nw36 t256 0 nch w=1u l=180n
M580 t256 nd13 0 0 nch w=1u l=180n
M581 t254 nw36 vdd vdd pch w=2u l=180n
M582 t254 t253 vdd vdd pch w=2u l=180n
CT257 t257 0 0.1f
M583 t254 nw36 t257 0 nch w=1u l=180n
M584 t257 t253 0 0 nch w=1u l=180n
M585 t255 nd13 vdd vdd pch w=2u l=180n
M586 t255 t253 vdd vdd pch w=2u l=180n
CT258 t258 0 0.1f
M587 t255 nd13 t258 0 nch w=1u l=180n
M588 t258 t253 0 0 nch w=1u l=180n
M589 nw37 t254 vdd vdd pch w=2u l=180n
M590 nw37 t255 vdd vdd pch w=2u l=180n
CT259 t259 0 0.1f
M591 nw37 t254 t259 0 nch w=1u l=180n
M592 t259 t255 0 0 nch w=1u l=180n
Cnw37 nw37 0 2f
CT260 t260 0 0.1f
CT261 t261 0 0.1f
CT262 t262 0 0.1f
M593 t260 nw37 vdd vdd pch w=2u l=180n
M594 t260 nd14 vdd vdd pch w=2u l=180n
CT263 t263 0 0.1f
M595 t260 nw37 t263 0 nch w=1u l=180n
M596 t263 nd14 0 0 nch w=1u l=180n
M597 t261 nw37 vdd vdd pch w=2u l=180n
M598 t261 t260 vdd vdd pch w=2u l=180n
CT264 t264 0 0.1f
M599 t261 nw37 t264 0 nch w=1u l=180n
M600 t264 t260 0 0 nch w=1u l=180n
M601 t262 nd14 vdd vdd pch w=2u l=180n
M602 t262 t260 vdd vdd pch w=2u l=180n
CT265 t265 0 0.1f
M603 t262 nd14 t265 0 nch w=1u l=180n
M604 t265 t260 0 0 nch w=1u l=180n
M605 nw38 t261 vdd vdd pch w=2u l=180n
M606 nw38 t262 vdd vdd pch w=2u l=180n
CT266 t266 0 0.1f
M607 nw38 t261 t266 0 nch w=1u l=180n
M608 t266 t262 0 0 nch w=1u l=180n
Cnw38 nw38 0 2f
CT267 t267 0 0.1f
CT268 t268 0 0.1f
CT269 t269 0 0.1f
M609 t267 nw38 vdd vdd pch w=2u l=180n
M610 t267 nd15 vdd vdd pch w=2u l=180n
CT270 t270 0 0.1f
M611 t267 nw38 t270 0 nch w=1u l=180n
M612 t270 nd15 0 0 nch w=1u l=180n
M613 t268 nw38 vdd vdd pch w=2u l=180n
M614 t268 t267 vdd vdd pch w=2u l=180n
CT271 t271 0 0.1f
M615 t268 nw38 t271 0 nch w=1u l=180n
M616 t271 t267 0 0 nch w=1u l=180n
M617 t269 nd15 vdd vdd pch w=2u l=180n
M618 t269 t267 vdd vdd pch w=2u l=180n
CT272 t272 0 0.1f
M619 t269 nd15 t272 0 nch w=1u l=180n
M620 t272 t267 0 0 nch w=1u l=180n
M621 nw39 t268 vdd vdd pch w=2u l=180n
M622 nw39 t269 vdd vdd pch w=2u l=180n
CT273 t273 0 0.1f
M623 nw39 t268 t273 0 nch w=1u l=180n
M624 t273 t269 0 0 nch w=1u l=180n
Cnw39 nw39 0 2f
CT274 t274 0 0.1f
CT275 t275 0 0.1f
CT276 t276 0 0.1f
M625 t274 nw39 vdd vdd pch w=2u l=180n
M626 t274 nr4 vdd vdd pch w=2u l=180n
CT277 t277 0 0.1f
M627 t274 nw39 t277 0 nch w=1u l=180n
M628 t277 nr4 0 0 nch w=1u l=180n
M629 t275 nw39 vdd vdd pch w=2u l=180n
M630 t275 t274 vdd vdd pch w=2u l=180n
CT278 t278 0 0.1f
M631 t275 nw39 t278 0 nch w=1u l=180n
M632 t278 t274 0 0 nch w=1u l=180n
M633 t276 nr4 vdd vdd pch w=2u l=180n
M634 t276 t274 vdd vdd pch w=2u l=180n
CT279 t279 0 0.1f
M635 t276 nr4 t279 0 nch w=1u l=180n
M636 t279 t274 0 0 nch w=1u l=180n
M637 nw40 t275 vdd vdd pch w=2u l=180n
M638 nw40 t276 vdd vdd pch w=2u l=180n
CT280 t280 0 0.1f
M639 nw40 t275 t280 0 nch w=1u l=180n
M640 t280 t276 0 0 nch w=1u l=180n
Cnw40 nw40 0 2f
M641 nw41 nw10 vdd vdd pch w=2u l=180n
M642 nw41 nw10 0 0 nch w=1u l=180n
Cnw41 nw41 0 2f
M643 nw42 nw19 vdd vdd pch w=2u l=180n
M644 nw42 nw19 0 0 nch w=1u l=180n
Cnw42 nw42 0 2f
M645 nw43 nw28 vdd vdd pch w=2u l=180n
M646 nw43 nw28 0 0 nch w=1u l=180n
Cnw43 nw43 0 2f
M647 nw44 nw35 vdd vdd pch w=2u l=180n
M648 nw44 nw35 0 0 nch w=1u l=180n
Cnw44 nw44 0 2f
M649 nw45 nw40 vdd vdd pch w=2u l=180n
M650 nw45 nw40 0 0 nch w=1u l=180n
Cnw45 nw45 0 2f
CT281 t281 0 0.1f
M651 t281 nw10 vdd vdd pch w=2u l=180n
M652 t281 nw19 vdd vdd pch w=2u l=180n
M653 t281 nw43 vdd vdd pch w=2u l=180n
M654 t281 nw44 vdd vdd pch w=2u l=180n
M655 t281 nw45 vdd vdd pch w=2u l=180n
M656 t281 nen vdd vdd pch w=2u l=180n
CT282 t282 0 0.1f
M657 t281 nw10 t282 0 nch w=1u l=180n
CT283 t283 0 0.1f
M658 t282 nw19 t283 0 nch w=1u l=180n
CT284 t284 0 0.1f
M659 t283 nw43 t284 0 nch w=1u l=180n
CT285 t285 0 0.1f
M660 t284 nw44 t285 0 nch w=1u l=180n
CT286 t286 0 0.1f
M661 t285 nw45 t286 0 nch w=1u l=180n
M662 t286 nen 0 0 nch w=1u l=180n
M663 nw46 t281 vdd vdd pch w=2u l=180n
M664 nw46 t281 0 0 nch w=1u l=180n
Cnw46 nw46 0 2f
CT287 t287 0 0.1f
CT288 t288 0 0.1f
CT289 t289 0 0.1f
M665 t287 nd0 vdd vdd pch w=2u l=180n
M666 t287 nw46 vdd vdd pch w=2u l=180n
CT290 t290 0 0.1f
M667 t287 nd0 t290 0 nch w=1u l=180n
M668 t290 nw46 0 0 nch w=1u l=180n
M669 t288 nd0 vdd vdd pch w=2u l=180n
M670 t288 t287 vdd vdd pch w=2u l=180n
CT291 t291 0 0.1f
M671 t288 nd0 t291 0 nch w=1u l=180n
M672 t291 t287 0 0 nch w=1u l=180n
M673 t289 nw46 vdd vdd pch w=2u l=180n
M674 t289 t287 vdd vdd pch w=2u l=180n
CT292 t292 0 0.1f
M675 t289 nw46 t292 0 nch w=1u l=180n
M676 t292 t287 0 0 nch w=1u l=180n
M677 nw47 t288 vdd vdd pch w=2u l=180n
M678 nw47 t289 vdd vdd pch w=2u l=180n
CT293 t293 0 0.1f
M679 nw47 t288 t293 0 nch w=1u l=180n
M680 t293 t289 0 0 nch w=1u l=180n
Cnw47 nw47 0 2f
CT294 t294 0 0.1f
M681 t294 nw47 vdd vdd pch w=2u l=180n
M682 t294 nw47 0 0 nch w=1u l=180n
M683 nq0 t294 vdd vdd pch w=2u l=180n
M684 nq0 t294 0 0 nch w=1u l=180n
Cnq0 nq0 0 2f
CT295 t295 0 0.1f
M685 t295 nw10 vdd vdd pch w=2u l=180n
M686 t295 nw42 vdd vdd pch w=2u l=180n
M687 t295 nw28 vdd vdd pch w=2u l=180n
M688 t295 nw44 vdd vdd pch w=2u l=180n
M689 t295 nw45 vdd vdd pch w=2u l=180n
M690 t295 nen vdd vdd pch w=2u l=180n
CT296 t296 0 0.1f
M691 t295 nw10 t296 0 nch w=1u l=180n
CT297 t297 0 0.1f
M692 t296 nw42 t297 0 nch w=1u l=180n
CT298 t298 0 0.1f
M693 t297 nw28 t298 0 nch w=1u l=180n
CT299 t299 0 0.1f
M694 t298 nw44 t299 0 nch w=1u l=180n
CT300 t300 0 0.1f
M695 t299 nw45 t300 0 nch w=1u l=180n
M696 t300 nen 0 0 nch w=1u l=180n
M697 nw49 t295 vdd vdd pch w=2u l=180n
M698 nw49 t295 0 0 nch w=1u l=180n
Cnw49 nw49 0 2f
CT301 t301 0 0.1f
CT302 t302 0 0.1f
CT303 t303 0 0.1f
M699 t301 nd1 vdd vdd pch w=2u l=180n
M700 t301 nw49 vdd vdd pch w=2u l=180n
CT304 t304 0 0.1f
M701 t301 nd1 t304 0 nch w=1u l=180n
M702 t304 nw49 0 0 nch w=1u l=180n
M703 t302 nd1 vdd vdd pch w=2u l=180n
M704 t302 t301 vdd vdd pch w=2u l=180n
CT305 t305 0 0.1f
M705 t302 nd1 t305 0 nch w=1u l=180n
M706 t305 t301 0 0 nch w=1u l=180n
M707 t303 nw49 vdd vdd pch w=2u l=180n
M708 t303 t301 vdd vdd pch w=2u l=180n
CT306 t306 0 0.1f
M709 t303 nw49 t306 0 nch w=1u l=180n
M710 t306 t301 0 0 nch w=1u l=180n
M711 nw50 t302 vdd vdd pch w=2u l=180n
M712 nw50 t303 vdd vdd pch w=2u l=180n
CT307 t307 0 0.1f
M713 nw50 t302 t307 0 nch w=1u l=180n
M714 t307 t303 0 0 nch w=1u l=180n
Cnw50 nw50 0 2f
CT308 t308 0 0.1f
M715 t308 nw50 vdd vdd pch w=2u l=180n
M716 t308 nw50 0 0 nch w=1u l=180n
M717 nq1 t308 vdd vdd pch w=2u l=180n
M718 nq1 t308 0 0 nch w=1u l=180n
Cnq1 nq1 0 2f
CT309 t309 0 0.1f
M719 t309 nw41 vdd vdd pch w=2u l=180n
M720 t309 nw19 vdd vdd pch w=2u l=180n
M721 t309 nw28 vdd vdd pch w=2u l=180n
M722 t309 nw44 vdd vdd pch w=2u l=180n
M723 t309 nw45 vdd vdd pch w=2u l=180n
M724 t309 nen vdd vdd pch w=2u l=180n
CT310 t310 0 0.1f
M725 t309 nw41 t310 0 nch w=1u l=180n
CT311 t311 0 0.1f
M726 t310 nw19 t311 0 nch w=1u l=180n
CT312 t312 0 0.1f
M727 t311 nw28 t312 0 nch w=1u l=180n
CT313 t313 0 0.1f
M728 t312 nw44 t313 0 nch w=1u l=180n
CT314 t314 0 0.1f
M729 t313 nw45 t314 0 nch w=1u l=180n
M730 t314 nen 0 0 nch w=1u l=180n
M731 nw52 t309 vdd vdd pch w=2u l=180n
M732 nw52 t309 0 0 nch w=1u l=180n
Cnw52 nw52 0 2f
CT315 t315 0 0.1f
CT316 t316 0 0.1f
CT317 t317 0 0.1f
M733 t315 nd2 vdd vdd pch w=2u l=180n
M734 t315 nw52 vdd vdd pch w=2u l=180n
CT318 t318 0 0.1f
M735 t315 nd2 t318 0 nch w=1u l=180n
M736 t318 nw52 0 0 nch w=1u l=180n
M737 t316 nd2 vdd vdd pch w=2u l=180n
M738 t316 t315 vdd vdd pch w=2u l=180n
CT319 t319 0 0.1f
M739 t316 nd2 t319 0 nch w=1u l=180n
M740 t319 t315 0 0 nch w=1u l=180n
M741 t317 nw52 vdd vdd pch w=2u l=180n
M742 t317 t315 vdd vdd pch w=2u l=180n
CT320 t320 0 0.1f
M743 t317 nw52 t320 0 nch w=1u l=180n
M744 t320 t315 0 0 nch w=1u l=180n
M745 nw53 t316 vdd vdd pch w=2u l=180n
M746 nw53 t317 vdd vdd pch w=2u l=180n
CT321 t321 0 0.1f
M747 nw53 t316 t321 0 nch w=1u l=180n
M748 t321 t317 0 0 nch w=1u l=180n
Cnw53 nw53 0 2f
CT322 t322 0 0.1f
M749 t322 nw53 vdd vdd pch w=2u l=180n
M750 t322 nw53 0 0 nch w=1u l=180n
M751 nq2 t322 vdd vdd pch w=2u l=180n
M752 nq2 t322 0 0 nch w=1u l=180n
Cnq2 nq2 0 2f
CT323 t323 0 0.1f
M753 t323 nw10 vdd vdd pch w=2u l=180n
M754 t323 nw19 vdd vdd pch w=2u l=180n
M755 t323 nw28 vdd vdd pch w=2u l=180n
M756 t323 nw44 vdd vdd pch w=2u l=180n
M757 t323 nw45 vdd vdd pch w=2u l=180n
M758 t323 nen vdd vdd pch w=2u l=180n
CT324 t324 0 0.1f
M759 t323 nw10 t324 0 nch w=1u l=180n
CT325 t325 0 0.1f
M760 t324 nw19 t325 0 nch w=1u l=180n
CT326 t326 0 0.1f
M761 t325 nw28 t326 0 nch w=1u l=180n
CT327 t327 0 0.1f
M762 t326 nw44 t327 0 nch w=1u l=180n
CT328 t328 0 0.1f
M763 t327 nw45 t328 0 nch w=1u l=180n
M764 t328 nen 0 0 nch w=1u l=180n
M765 nw55 t323 vdd vdd pch w=2u l=180n
M766 nw55 t323 0 0 nch w=1u l=180n
Cnw55 nw55 0 2f
CT329 t329 0 0.1f
CT330 t330 0 0.1f
CT331 t331 0 0.1f
M767 t329 nd3 vdd vdd pch w=2u l=180n
M768 t329 nw55 vdd vdd pch w=2u l=180n
CT332 t332 0 0.1f
M769 t329 nd3 t332 0 nch w=1u l=180n
M770 t332 nw55 0 0 nch w=1u l=180n
M771 t330 nd3 vdd vdd pch w=2u l=180n
M772 t330 t329 vdd vdd pch w=2u l=180n
CT333 t333 0 0.1f
M773 t330 nd3 t333 0 nch w=1u l=180n
M774 t333 t329 0 0 nch w=1u l=180n
M775 t331 nw55 vdd vdd pch w=2u l=180n
M776 t331 t329 vdd vdd pch w=2u l=180n
CT334 t334 0 0.1f
M777 t331 nw55 t334 0 nch w=1u l=180n
M778 t334 t329 0 0 nch w=1u l=180n
M779 nw56 t330 vdd vdd pch w=2u l=180n
M780 nw56 t331 vdd vdd pch w=2u l=180n
CT335 t335 0 0.1f
M781 nw56 t330 t335 0 nch w=1u l=180n
M782 t335 t331 0 0 nch w=1u l=180n
Cnw56 nw56 0 2f
CT336 t336 0 0.1f
M783 t336 nw56 vdd vdd pch w=2u l=180n
M784 t336 nw56 0 0 nch w=1u l=180n
M785 nq3 t336 vdd vdd pch w=2u l=180n
M786 nq3 t336 0 0 nch w=1u l=180n
Cnq3 nq3 0 2f
CT337 t337 0 0.1f
M787 t337 nw10 vdd vdd pch w=2u l=180n
M788 t337 nw42 vdd vdd pch w=2u l=180n
M789 t337 nw43 vdd vdd pch w=2u l=180n
M790 t337 nw35 vdd vdd pch w=2u l=180n
M791 t337 nw45 vdd vdd pch w=2u l=180n
M792 t337 nen vdd vdd pch w=2u l=180n
CT338 t338 0 0.1f
M793 t337 nw10 t338 0 nch w=1u l=180n
CT339 t339 0 0.1f
M794 t338 nw42 t339 0 nch w=1u l=180n
CT340 t340 0 0.1f
M795 t339 nw43 t340 0 nch w=1u l=180n
CT341 t341 0 0.1f
M796 t340 nw35 t341 0 nch w=1u l=180n
CT342 t342 0 0.1f
M797 t341 nw45 t342 0 nch w=1u l=180n
M798 t342 nen 0 0 nch w=1u l=180n
M799 nw58 t337 vdd vdd pch w=2u l=180n
M800 nw58 t337 0 0 nch w=1u l=180n
Cnw58 nw58 0 2f
CT343 t343 0 0.1f
CT344 t344 0 0.1f
CT345 t345 0 0.1f
M801 t343 nd4 vdd vdd pch w=2u l=180n
M802 t343 nw58 vdd vdd pch w=2u l=180n
CT346 t346 0 0.1f
M803 t343 nd4 t346 0 nch w=1u l=180n
M804 t346 nw58 0 0 nch w=1u l=180n
M805 t344 nd4 vdd vdd pch w=2u l=180n
M806 t344 t343 vdd vdd pch w=2u l=180n
CT347 t347 0 0.1f
M807 t344 nd4 t347 0 nch w=1u l=180n
M808 t347 t343 0 0 nch w=1u l=180n
M809 t345 nw58 vdd vdd pch w=2u l=180n
M810 t345 t343 vdd vdd pch w=2u l=180n
CT348 t348 0 0.1f
M811 t345 nw58 t348 0 nch w=1u l=180n
M812 t348 t343 0 0 nch w=1u l=180n
M813 nw59 t344 vdd vdd pch w=2u l=180n
M814 nw59 t345 vdd vdd pch w=2u l=180n
CT349 t349 0 0.1f
M815 nw59 t344 t349 0 nch w=1u l=180n
M816 t349 t345 0 0 nch w=1u l=180n
Cnw59 nw59 0 2f
CT350 t350 0 0.1f
M817 t350 nw59 vdd vdd pch w=2u l=180n
M818 t350 nw59 0 0 nch w=1u l=180n
M819 nq4 t350 vdd vdd pch w=2u l=180n
M820 nq4 t350 0 0 nch w=1u l=180n
Cnq4 nq4 0 2f
CT351 t351 0 0.1f
M821 t351 nw41 vdd vdd pch w=2u l=180n
M822 t351 nw19 vdd vdd pch w=2u l=180n
M823 t351 nw43 vdd vdd pch w=2u l=180n
M824 t351 nw35 vdd vdd pch w=2u l=180n
M825 t351 nw45 vdd vdd pch w=2u l=180n
M826 t351 nen vdd vdd pch w=2u l=180n
CT352 t352 0 0.1f
M827 t351 nw41 t352 0 nch w=1u l=180n
CT353 t353 0 0.1f
M828 t352 nw19 t353 0 nch w=1u l=180n
CT354 t354 0 0.1f
M829 t353 nw43 t354 0 nch w=1u l=180n
CT355 t355 0 0.1f
M830 t354 nw35 t355 0 nch w=1u l=180n
CT356 t356 0 0.1f
M831 t355 nw45 t356 0 nch w=1u l=180n
M832 t356 nen 0 0 nch w=1u l=180n
M833 nw61 t351 vdd vdd pch w=2u l=180n
M834 nw61 t351 0 0 nch w=1u l=180n
Cnw61 nw61 0 2f
CT357 t357 0 0.1f
CT358 t358 0 0.1f
CT359 t359 0 0.1f
M835 t357 nd5 vdd vdd pch w=2u l=180n
M836 t357 nw61 vdd vdd pch w=2u l=180n
CT360 t360 0 0.1f
M837 t357 nd5 t360 0 nch w=1u l=180n
M838 t360 nw61 0 0 nch w=1u l=180n
M839 t358 nd5 vdd vdd pch w=2u l=180n
M840 t358 t357 vdd vdd pch w=2u l=180n
CT361 t361 0 0.1f
M841 t358 nd5 t361 0 nch w=1u l=180n
M842 t361 t357 0 0 nch w=1u l=180n
M843 t359 nw61 vdd vdd pch w=2u l=180n
M844 t359 t357 vdd vdd pch w=2u l=180n
CT362 t362 0 0.1f
M845 t359 nw61 t362 0 nch w=1u l=180n
M846 t362 t357 0 0 nch w=1u l=180n
M847 nw62 t358 vdd vdd pch w=2u l=180n
M848 nw62 t359 vdd vdd pch w=2u l=180n
CT363 t363 0 0.1f
M849 nw62 t358 t363 0 nch w=1u l=180n
M850 t363 t359 0 0 nch w=1u l=180n
Cnw62 nw62 0 2f
CT364 t364 0 0.1f
M851 t364 nw62 vdd vdd pch w=2u l=180n
M852 t364 nw62 0 0 nch w=1u l=180n
M853 nq5 t364 vdd vdd pch w=2u l=180n
M854 nq5 t364 0 0 nch w=1u l=180n
Cnq5 nq5 0 2f
CT365 t365 0 0.1f
M855 t365 nw10 vdd vdd pch w=2u l=180n
M856 t365 nw19 vdd vdd pch w=2u l=180n
M857 t365 nw43 vdd vdd pch w=2u l=180n
M858 t365 nw35 vdd vdd pch w=2u l=180n
M859 t365 nw45 vdd vdd pch w=2u l=180n
M860 t365 nen vdd vdd pch w=2u l=180n
CT366 t366 0 0.1f
M861 t365 nw10 t366 0 nch w=1u l=180n
CT367 t367 0 0.1f
M862 t366 nw19 t367 0 nch w=1u l=180n
CT368 t368 0 0.1f
M863 t367 nw43 t368 0 nch w=1u l=180n
CT369 t369 0 0.1f
M864 t368 nw35 t369 0 nch w=1u l=180n
CT370 t370 0 0.1f
M865 t369 nw45 t370 0 nch w=1u l=180n
M866 t370 nen 0 0 nch w=1u l=180n
M867 nw64 t365 vdd vdd pch w=2u l=180n
M868 nw64 t365 0 0 nch w=1u l=180n
Cnw64 nw64 0 2f
CT371 t371 0 0.1f
CT372 t372 0 0.1f
CT373 t373 0 0.1f
M869 t371 nd6 vdd vdd pch w=2u l=180n
M870 t371 nw64 vdd vdd pch w=2u l=180n
CT374 t374 0 0.1f
M871 t371 nd6 t374 0 nch w=1u l=180n
M872 t374 nw64 0 0 nch w=1u l=180n
M873 t372 nd6 vdd vdd pch w=2u l=180n
M874 t372 t371 vdd vdd pch w=2u l=180n
CT375 t375 0 0.1f
M875 t372 nd6 t375 0 nch w=1u l=180n
M876 t375 t371 0 0 nch w=1u l=180n
M877 t373 nw64 vdd vdd pch w=2u l=180n
M878 t373 t371 vdd vdd pch w=2u l=180n
CT376 t376 0 0.1f
M879 t373 nw64 t376 0 nch w=1u l=180n
M880 t376 t371 0 0 nch w=1u l=180n
M881 nw65 t372 vdd vdd pch w=2u l=180n
M882 nw65 t373 vdd vdd pch w=2u l=180n
CT377 t377 0 0.1f
M883 nw65 t372 t377 0 nch w=1u l=180n
M884 t377 t373 0 0 nch w=1u l=180n
Cnw65 nw65 0 2f
CT378 t378 0 0.1f
M885 t378 nw65 vdd vdd pch w=2u l=180n
M886 t378 nw65 0 0 nch w=1u l=180n
M887 nq6 t378 vdd vdd pch w=2u l=180n
M888 nq6 t378 0 0 nch w=1u l=180n
Cnq6 nq6 0 2f
CT379 t379 0 0.1f
M889 t379 nw41 vdd vdd pch w=2u l=180n
M890 t379 nw42 vdd vdd pch w=2u l=180n
M891 t379 nw28 vdd vdd pch w=2u l=180n
M892 t379 nw35 vdd vdd pch w=2u l=180n
M893 t379 nw45 vdd vdd pch w=2u l=180n
M894 t379 nen vdd vdd pch w=2u l=180n
CT380 t380 0 0.1f
M895 t379 nw41 t380 0 nch w=1u l=180n
CT381 t381 0 0.1f
M896 t380 nw42 t381 0 nch w=1u l=180n
CT382 t382 0 0.1f
M897 t381 nw28 t382 0 nch w=1u l=180n
CT383 t383 0 0.1f
M898 t382 nw35 t383 0 nch w=1u l=180n
CT384 t384 0 0.1f
M899 t383 nw45 t384 0 nch w=1u l=180n
M900 t384 nen 0 0 nch w=1u l=180n
M901 nw67 t379 vdd vdd pch w=2u l=180n
M902 nw67 t379 0 0 nch w=1u l=180n
Cnw67 nw67 0 2f
CT385 t385 0 0.1f
CT386 t386 0 0.1f
CT387 t387 0 0.1f
M903 t385 nd7 vdd vdd pch w=2u l=180n
M904 t385 nw67 vdd vdd pch w=2u l=180n
CT388 t388 0 0.1f
M905 t385 nd7 t388 0 nch w=1u l=180n
M906 t388 nw67 0 0 nch w=1u l=180n
M907 t386 nd7 vdd vdd pch w=2u l=180n
M908 t386 t385 vdd vdd pch w=2u l=180n
CT389 t389 0 0.1f
M909 t386 nd7 t389 0 nch w=1u l=180n
M910 t389 t385 0 0 nch w=1u l=180n
M911 t387 nw67 vdd vdd pch w=2u l=180n
M912 t387 t385 vdd vdd pch w=2u l=180n
CT390 t390 0 0.1f
M913 t387 nw67 t390 0 nch w=1u l=180n
M914 t390 t385 0 0 nch w=1u l=180n
M915 nw68 t386 vdd vdd pch w=2u l=180n
M916 nw68 t387 vdd vdd pch w=2u l=180n
CT391 t391 0 0.1f
M917 nw68 t386 t391 0 nch w=1u l=180n
M918 t391 t387 0 0 nch w=1u l=180n
Cnw68 nw68 0 2f
CT392 t392 0 0.1f
M919 t392 nw68 vdd vdd pch w=2u l=180n
M920 t392 nw68 0 0 nch w=1u l=180n
M921 nq7 t392 vdd vdd pch w=2u l=180n
M922 nq7 t392 0 0 nch w=1u l=180n
Cnq7 nq7 0 2f
CT393 t393 0 0.1f
M923 t393 nw10 vdd vdd pch w=2u l=180n
M924 t393 nw42 vdd vdd pch w=2u l=180n
M925 t393 nw28 vdd vdd pch w=2u l=180n
M926 t393 nw35 vdd vdd pch w=2u l=180n
M927 t393 nw45 vdd vdd pch w=2u l=180n
M928 t393 nen vdd vdd pch w=2u l=180n
CT394 t394 0 0.1f
M929 t393 nw10 t394 0 nch w=1u l=180n
CT395 t395 0 0.1f
M930 t394 nw42 t395 0 nch w=1u l=180n
CT396 t396 0 0.1f
M931 t395 nw28 t396 0 nch w=1u l=180n
CT397 t397 0 0.1f
M932 t396 nw35 t397 0 nch w=1u l=180n
CT398 t398 0 0.1f
M933 t397 nw45 t398 0 nch w=1u l=180n
M934 t398 nen 0 0 nch w=1u l=180n
M935 nw70 t393 vdd vdd pch w=2u l=180n
M936 nw70 t393 0 0 nch w=1u l=180n
Cnw70 nw70 0 2f
CT399 t399 0 0.1f
CT400 t400 0 0.1f
CT401 t401 0 0.1f
M937 t399 nd8 vdd vdd pch w=2u l=180n
M938 t399 nw70 vdd vdd pch w=2u l=180n
CT402 t402 0 0.1f
M939 t399 nd8 t402 0 nch w=1u l=180n
M940 t402 nw70 0 0 nch w=1u l=180n
M941 t400 nd8 vdd vdd pch w=2u l=180n
M942 t400 t399 vdd vdd pch w=2u l=180n
CT403 t403 0 0.1f
M943 t400 nd8 t403 0 nch w=1u l=180n
M944 t403 t399 0 0 nch w=1u l=180n
M945 t401 nw70 vdd vdd pch w=2u l=180n
M946 t401 t399 vdd vdd pch w=2u l=180n
CT404 t404 0 0.1f
M947 t401 nw70 t404 0 nch w=1u l=180n
M948 t404 t399 0 0 nch w=1u l=180n
M949 nw71 t400 vdd vdd pch w=2u l=180n
M950 nw71 t401 vdd vdd pch w=2u l=180n
CT405 t405 0 0.1f
M951 nw71 t400 t405 0 nch w=1u l=180n
M952 t405 t401 0 0 nch w=1u l=180n
Cnw71 nw71 0 2f
CT406 t406 0 0.1f
M953 t406 nw71 vdd vdd pch w=2u l=180n
M954 t406 nw71 0 0 nch w=1u l=180n
M955 nq8 t406 vdd vdd pch w=2u l=180n
M956 nq8 t406 0 0 nch w=1u l=180n
Cnq8 nq8 0 2f
CT407 t407 0 0.1f
M957 t407 nw41 vdd vdd pch w=2u l=180n
M958 t407 nw19 vdd vdd pch w=2u l=180n
M959 t407 nw28 vdd vdd pch w=2u l=180n
M960 t407 nw35 vdd vdd pch w=2u l=180n
M961 t407 nw45 vdd vdd pch w=2u l=180n
M962 t407 nen vdd vdd pch w=2u l=180n
CT408 t408 0 0.1f
M963 t407 nw41 t408 0 nch w=1u l=180n
CT409 t409 0 0.1f
M964 t408 nw19 t409 0 nch w=1u l=180n
CT410 t410 0 0.1f
M965 t409 nw28 t410 0 nch w=1u l=180n
CT411 t411 0 0.1f
M966 t410 nw35 t411 0 nch w=1u l=180n
CT412 t412 0 0.1f
M967 t411 nw45 t412 0 nch w=1u l=180n
M968 t412 nen 0 0 nch w=1u l=180n
M969 nw73 t407 vdd vdd pch w=2u l=180n
M970 nw73 t407 0 0 nch w=1u l=180n
Cnw73 nw73 0 2f
CT413 t413 0 0.1f
CT414 t414 0 0.1f
CT415 t415 0 0.1f
M971 t413 nd9 vdd vdd pch w=2u l=180n
M972 t413 nw73 vdd vdd pch w=2u l=180n
CT416 t416 0 0.1f
M973 t413 nd9 t416 0 nch w=1u l=180n
M974 t416 nw73 0 0 nch w=1u l=180n
M975 t414 nd9 vdd vdd pch w=2u l=180n
M976 t414 t413 vdd vdd pch w=2u l=180n
CT417 t417 0 0.1f
M977 t414 nd9 t417 0 nch w=1u l=180n
M978 t417 t413 0 0 nch w=1u l=180n
M979 t415 nw73 vdd vdd pch w=2u l=180n
M980 t415 t413 vdd vdd pch w=2u l=180n
CT418 t418 0 0.1f
M981 t415 nw73 t418 0 nch w=1u l=180n
M982 t418 t413 0 0 nch w=1u l=180n
M983 nw74 t414 vdd vdd pch w=2u l=180n
M984 nw74 t415 vdd vdd pch w=2u l=180n
CT419 t419 0 0.1f
M985 nw74 t414 t419 0 nch w=1u l=180n
M986 t419 t415 0 0 nch w=1u l=180n
Cnw74 nw74 0 2f
CT420 t420 0 0.1f
M987 t420 nw74 vdd vdd pch w=2u l=180n
M988 t420 nw74 0 0 nch w=1u l=180n
M989 nq9 t420 vdd vdd pch w=2u l=180n
M990 nq9 t420 0 0 nch w=1u l=180n
Cnq9 nq9 0 2f
CT421 t421 0 0.1f
M991 t421 nw10 vdd vdd pch w=2u l=180n
M992 t421 nw19 vdd vdd pch w=2u l=180n
M993 t421 nw28 vdd vdd pch w=2u l=180n
M994 t421 nw35 vdd vdd pch w=2u l=180n
M995 t421 nw45 vdd vdd pch w=2u l=180n
M996 t421 nen vdd vdd pch w=2u l=180n
CT422 t422 0 0.1f
M997 t421 nw10 t422 0 nch w=1u l=180n
CT423 t423 0 0.1f
M998 t422 nw19 t423 0 nch w=1u l=180n
CT424 t424 0 0.1f
M999 t423 nw28 t424 0 nch w=1u l=180n
CT425 t425 0 0.1f
M1000 t424 nw35 t425 0 nch w=1u l=180n
CT426 t426 0 0.1f
M1001 t425 nw45 t426 0 nch w=1u l=180n
M1002 t426 nen 0 0 nch w=1u l=180n
M1003 nw76 t421 vdd vdd pch w=2u l=180n
M1004 nw76 t421 0 0 nch w=1u l=180n
Cnw76 nw76 0 2f
CT427 t427 0 0.1f
CT428 t428 0 0.1f
CT429 t429 0 0.1f
M1005 t427 nd10 vdd vdd pch w=2u l=180n
M1006 t427 nw76 vdd vdd pch w=2u l=180n
CT430 t430 0 0.1f
M1007 t427 nd10 t430 0 nch w=1u l=180n
M1008 t430 nw76 0 0 nch w=1u l=180n
M1009 t428 nd10 vdd vdd pch w=2u l=180n
M1010 t428 t427 vdd vdd pch w=2u l=180n
CT431 t431 0 0.1f
M1011 t428 nd10 t431 0 nch w=1u l=180n
M1012 t431 t427 0 0 nch w=1u l=180n
M1013 t429 nw76 vdd vdd pch w=2u l=180n
M1014 t429 t427 vdd vdd pch w=2u l=180n
CT432 t432 0 0.1f
M1015 t429 nw76 t432 0 nch w=1u l=180n
M1016 t432 t427 0 0 nch w=1u l=180n
M1017 nw77 t428 vdd vdd pch w=2u l=180n
M1018 nw77 t429 vdd vdd pch w=2u l=180n
CT433 t433 0 0.1f
M1019 nw77 t428 t433 0 nch w=1u l=180n
M1020 t433 t429 0 0 nch w=1u l=180n
Cnw77 nw77 0 2f
CT434 t434 0 0.1f
M1021 t434 nw77 vdd vdd pch w=2u l=180n
M1022 t434 nw77 0 0 nch w=1u l=180n
M1023 nq10 t434 vdd vdd pch w=2u l=180n
M1024 nq10 t434 0 0 nch w=1u l=180n
Cnq10 nq10 0 2f
CT435 t435 0 0.1f
M1025 t435 nw10 vdd vdd pch w=2u l=180n
M1026 t435 nw42 vdd vdd pch w=2u l=180n
M1027 t435 nw43 vdd vdd pch w=2u l=180n
M1028 t435 nw44 vdd vdd pch w=2u l=180n
M1029 t435 nw40 vdd vdd pch w=2u l=180n
M1030 t435 nen vdd vdd pch w=2u l=180n
CT436 t436 0 0.1f
M1031 t435 nw10 t436 0 nch w=1u l=180n
CT437 t437 0 0.1f
M1032 t436 nw42 t437 0 nch w=1u l=180n
CT438 t438 0 0.1f
M1033 t437 nw43 t438 0 nch w=1u l=180n
CT439 t439 0 0.1f
M1034 t438 nw44 t439 0 nch w=1u l=180n
CT440 t440 0 0.1f
M1035 t439 nw40 t440 0 nch w=1u l=180n
M1036 t440 nen 0 0 nch w=1u l=180n
M1037 nw79 t435 vdd vdd pch w=2u l=180n
M1038 nw79 t435 0 0 nch w=1u l=180n
Cnw79 nw79 0 2f
CT441 t441 0 0.1f
CT442 t442 0 0.1f
CT443 t443 0 0.1f
M1039 t441 nd11 vdd vdd pch w=2u l=180n
M1040 t441 nw79 vdd vdd pch w=2u l=180n
CT444 t444 0 0.1f
M1041 t441 nd11 t444 0 nch w=1u l=180n
M1042 t444 nw79 0 0 nch w=1u l=180n
M1043 t442 nd11 vdd vdd pch w=2u l=180n
M1044 t442 t441 vdd vdd pch w=2u l=180n
CT445 t445 0 0.1f
M1045 t442 nd11 t445 0 nch w=1u l=180n
M1046 t445 t441 0 0 nch w=1u l=180n
M1047 t443 nw79 vdd vdd pch w=2u l=180n
M1048 t443 t441 vdd vdd pch w=2u l=180n
CT446 t446 0 0.1f
M1049 t443 nw79 t446 0 nch w=1u l=180n
M1050 t446 t441 0 0 nch w=1u l=180n
M1051 nw80 t442 vdd vdd pch w=2u l=180n
M1052 nw80 t443 vdd vdd pch w=2u l=180n
CT447 t447 0 0.1f
M1053 nw80 t442 t447 0 nch w=1u l=180n
M1054 t447 t443 0 0 nch w=1u l=180n
Cnw80 nw80 0 2f
CT448 t448 0 0.1f
M1055 t448 nw80 vdd vdd pch w=2u l=180n
M1056 t448 nw80 0 0 nch w=1u l=180n
M1057 nq11 t448 vdd vdd pch w=2u l=180n
M1058 nq11 t448 0 0 nch w=1u l=180n
Cnq11 nq11 0 2f
CT449 t449 0 0.1f
M1059 t449 nw41 vdd vdd pch w=2u l=180n
M1060 t449 nw19 vdd vdd pch w=2u l=180n
M1061 t449 nw43 vdd vdd pch w=2u l=180n
M1062 t449 nw44 vdd vdd pch w=2u l=180n
M1063 t449 nw40 vdd vdd pch w=2u l=180n
M1064 t449 nen vdd vdd pch w=2u l=180n
CT450 t450 0 0.1f
M1065 t449 nw41 t450 0 nch w=1u l=180n
CT451 t451 0 0.1f
M1066 t450 nw19 t451 0 nch w=1u l=180n
CT452 t452 0 0.1f
M1067 t451 nw43 t452 0 nch w=1u l=180n
CT453 t453 0 0.1f
M1068 t452 nw44 t453 0 nch w=1u l=180n
CT454 t454 0 0.1f
M1069 t453 nw40 t454 0 nch w=1u l=180n
M1070 t454 nen 0 0 nch w=1u l=180n
M1071 nw82 t449 vdd vdd pch w=2u l=180n
M1072 nw82 t449 0 0 nch w=1u l=180n
Cnw82 nw82 0 2f
CT455 t455 0 0.1f
CT456 t456 0 0.1f
CT457 t457 0 0.1f
M1073 t455 nd12 vdd vdd pch w=2u l=180n
M1074 t455 nw82 vdd vdd pch w=2u l=180n
CT458 t458 0 0.1f
M1075 t455 nd12 t458 0 nch w=1u l=180n
M1076 t458 nw82 0 0 nch w=1u l=180n
M1077 t456 nd12 vdd vdd pch w=2u l=180n
M1078 t456 t455 vdd vdd pch w=2u l=180n
CT459 t459 0 0.1f
M1079 t456 nd12 t459 0 nch w=1u l=180n
M1080 t459 t455 0 0 nch w=1u l=180n
M1081 t457 nw82 vdd vdd pch w=2u l=180n
M1082 t457 t455 vdd vdd pch w=2u l=180n
CT460 t460 0 0.1f
M1083 t457 nw82 t460 0 nch w=1u l=180n
M1084 t460 t455 0 0 nch w=1u l=180n
M1085 nw83 t456 vdd vdd pch w=2u l=180n
M1086 nw83 t457 vdd vdd pch w=2u l=180n
CT461 t461 0 0.1f
M1087 nw83 t456 t461 0 nch w=1u l=180n
M1088 t461 t457 0 0 nch w=1u l=180n
Cnw83 nw83 0 2f
CT462 t462 0 0.1f
M1089 t462 nw83 vdd vdd pch w=2u l=180n
M1090 t462 nw83 0 0 nch w=1u l=180n
M1091 nq12 t462 vdd vdd pch w=2u l=180n
M1092 nq12 t462 0 0 nch w=1u l=180n
Cnq12 nq12 0 2f
CT463 t463 0 0.1f
M1093 t463 nw10 vdd vdd pch w=2u l=180n
M1094 t463 nw19 vdd vdd pch w=2u l=180n
M1095 t463 nw43 vdd vdd pch w=2u l=180n
M1096 t463 nw44 vdd vdd pch w=2u l=180n
M1097 t463 nw40 vdd vdd pch w=2u l=180n
M1098 t463 nen vdd vdd pch w=2u l=180n
CT464 t464 0 0.1f
M1099 t463 nw10 t464 0 nch w=1u l=180n
CT465 t465 0 0.1f
M1100 t464 nw19 t465 0 nch w=1u l=180n
CT466 t466 0 0.1f
M1101 t465 nw43 t466 0 nch w=1u l=180n
CT467 t467 0 0.1f
M1102 t466 nw44 t467 0 nch w=1u l=180n
CT468 t468 0 0.1f
M1103 t467 nw40 t468 0 nch w=1u l=180n
M1104 t468 nen 0 0 nch w=1u l=180n
M1105 nw85 t463 vdd vdd pch w=2u l=180n
M1106 nw85 t463 0 0 nch w=1u l=180n
Cnw85 nw85 0 2f
CT469 t469 0 0.1f
CT470 t470 0 0.1f
CT471 t471 0 0.1f
M1107 t469 nd13 vdd vdd pch w=2u l=180n
M1108 t469 nw85 vdd vdd pch w=2u l=180n
CT472 t472 0 0.1f
M1109 t469 nd13 t472 0 nch w=1u l=180n
M1110 t472 nw85 0 0 nch w=1u l=180n
M1111 t470 nd13 vdd vdd pch w=2u l=180n
M1112 t470 t469 vdd vdd pch w=2u l=180n
CT473 t473 0 0.1f
M1113 t470 nd13 t473 0 nch w=1u l=180n
M1114 t473 t469 0 0 nch w=1u l=180n
M1115 t471 nw85 vdd vdd pch w=2u l=180n
M1116 t471 t469 vdd vdd pch w=2u l=180n
CT474 t474 0 0.1f
M1117 t471 nw85 t474 0 nch w=1u l=180n
M1118 t474 t469 0 0 nch w=1u l=180n
M1119 nw86 t470 vdd vdd pch w=2u l=180n
M1120 nw86 t471 vdd vdd pch w=2u l=180n
CT475 t475 0 0.1f
M1121 nw86 t470 t475 0 nch w=1u l=180n
M1122 t475 t471 0 0 nch w=1u l=180n
Cnw86 nw86 0 2f
CT476 t476 0 0.1f
M1123 t476 nw86 vdd vdd pch w=2u l=180n
M1124 t476 nw86 0 0 nch w=1u l=180n
M1125 nq13 t476 vdd vdd pch w=2u l=180n
M1126 nq13 t476 0 0 nch w=1u l=180n
Cnq13 nq13 0 2f
CT477 t477 0 0.1f
M1127 t477 nw41 vdd vdd pch w=2u l=180n
M1128 t477 nw42 vdd vdd pch w=2u l=180n
M1129 t477 nw28 vdd vdd pch w=2u l=180n
M1130 t477 nw44 vdd vdd pch w=2u l=180n
M1131 t477 nw40 vdd vdd pch w=2u l=180n
M1132 t477 nen vdd vdd pch w=2u l=180n
CT478 t478 0 0.1f
M1133 t477 nw41 t478 0 nch w=1u l=180n
CT479 t479 0 0.1f
M1134 t478 nw42 t479 0 nch w=1u l=180n
CT480 t480 0 0.1f
M1135 t479 nw28 t480 0 nch w=1u l=180n
CT481 t481 0 0.1f
M1136 t480 nw44 t481 0 nch w=1u l=180n
CT482 t482 0 0.1f
M1137 t481 nw40 t482 0 nch w=1u l=180n
M1138 t482 nen 0 0 nch w=1u l=180n
M1139 nw88 t477 vdd vdd pch w=2u l=180n
M1140 nw88 t477 0 0 nch w=1u l=180n
Cnw88 nw88 0 2f
CT483 t483 0 0.1f
CT484 t484 0 0.1f
CT485 t485 0 0.1f
M1141 t483 nd14 vdd vdd pch w=2u l=180n
M1142 t483 nw88 vdd vdd pch w=2u l=180n
CT486 t486 0 0.1f
M1143 t483 nd14 t486 0 nch w=1u l=180n
M1144 t486 nw88 0 0 nch w=1u l=180n
M1145 t484 nd14 vdd vdd pch w=2u l=180n
M1146 t484 t483 vdd vdd pch w=2u l=180n
CT487 t487 0 0.1f
M1147 t484 nd14 t487 0 nch w=1u l=180n
M1148 t487 t483 0 0 nch w=1u l=180n
M1149 t485 nw88 vdd vdd pch w=2u l=180n
M1150 t485 t483 vdd vdd pch w=2u l=180n
CT488 t488 0 0.1f
M1151 t485 nw88 t488 0 nch w=1u l=180n
M1152 t488 t483 0 0 nch w=1u l=180n
M1153 nw89 t484 vdd vdd pch w=2u l=180n
M1154 nw89 t485 vdd vdd pch w=2u l=180n
CT489 t489 0 0.1f
M1155 nw89 t484 t489 0 nch w=1u l=180n
M1156 t489 t485 0 0 nch w=1u l=180n
Cnw89 nw89 0 2f
CT490 t490 0 0.1f
M1157 t490 nw89 vdd vdd pch w=2u l=180n
M1158 t490 nw89 0 0 nch w=1u l=180n
M1159 nq14 t490 vdd vdd pch w=2u l=180n
M1160 nq14 t490 0 0 nch w=1u l=180n
Cnq14 nq14 0 2f
CT491 t491 0 0.1f
M1161 t491 nw10 vdd vdd pch w=2u l=180n
M1162 t491 nw42 vdd vdd pch w=2u l=180n
M1163 t491 nw28 vdd vdd pch w=2u l=180n
M1164 t491 nw44 vdd vdd pch w=2u l=180n
M1165 t491 nw40 vdd vdd pch w=2u l=180n
M1166 t491 nen vdd vdd pch w=2u l=180n
CT492 t492 0 0.1f
M1167 t491 nw10 t492 0 nch w=1u l=180n
CT493 t493 0 0.1f
M1168 t492 nw42 t493 0 nch w=1u l=180n
CT494 t494 0 0.1f
M1169 t493 nw28 t494 0 nch w=1u l=180n
CT495 t495 0 0.1f
M1170 t494 nw44 t495 0 nch w=1u l=180n
CT496 t496 0 0.1f
M1171 t495 nw40 t496 0 nch w=1u l=180n
M1172 t496 nen 0 0 nch w=1u l=180n
M1173 nw91 t491 vdd vdd pch w=2u l=180n
M1174 nw91 t491 0 0 nch w=1u l=180n
Cnw91 nw91 0 2f
CT497 t497 0 0.1f
CT498 t498 0 0.1f
CT499 t499 0 0.1f
M1175 t497 nd15 vdd vdd pch w=2u l=180n
M1176 t497 nw91 vdd vdd pch w=2u l=180n
CT500 t500 0 0.1f
M1177 t497 nd15 t500 0 nch w=1u l=180n
M1178 t500 nw91 0 0 nch w=1u l=180n
M1179 t498 nd15 vdd vdd pch w=2u l=180n
M1180 t498 t497 vdd vdd pch w=2u l=180n
CT501 t501 0 0.1f
M1181 t498 nd15 t501 0 nch w=1u l=180n
M1182 t501 t497 0 0 nch w=1u l=180n
M1183 t499 nw91 vdd vdd pch w=2u l=180n
M1184 t499 t497 vdd vdd pch w=2u l=180n
CT502 t502 0 0.1f
M1185 t499 nw91 t502 0 nch w=1u l=180n
M1186 t502 t497 0 0 nch w=1u l=180n
M1187 nw92 t498 vdd vdd pch w=2u l=180n
M1188 nw92 t499 vdd vdd pch w=2u l=180n
CT503 t503 0 0.1f
M1189 nw92 t498 t503 0 nch w=1u l=180n
M1190 t503 t499 0 0 nch w=1u l=180n
Cnw92 nw92 0 2f
CT504 t504 0 0.1f
M1191 t504 nw92 vdd vdd pch w=2u l=180n
M1192 t504 nw92 0 0 nch w=1u l=180n
M1193 nq15 t504 vdd vdd pch w=2u l=180n
M1194 nq15 t504 0 0 nch w=1u l=180n
Cnq15 nq15 0 2f
.model nch NMOS (vto=0.45 kp=200u lambda=0.05)
.model pch PMOS (vto=-0.45 kp=100u lambda=0.05)
* outputs: nq0 nq1 nq2 nq3 nq4 nq5 nq6 nq7 nq8 nq9 nq10 nq11 nq12 nq13 nq14 nq15
.end
